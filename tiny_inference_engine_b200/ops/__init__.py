"""Python faces of the CUDA kernels: shape and dtype checks, then one launch on the current stream.

Tensors are torch CUDA tensors used as typed device memory; nothing here computes with torch.
"""
from __future__ import annotations

import os

import torch

from ..errors import InvalidArgument
from . import library
from .library import call, check_device

F32, BF16 = 0, 1
_DT = {torch.float32: F32, torch.bfloat16: BF16}


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise InvalidArgument(f"dtype {t.dtype} is not one of float32, bfloat16") from None


_RAW_STREAM = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_DEVICE_INDEX = None


def _stream() -> int:
    """The current stream's handle. (torch.cuda.current_stream() builds a Stream object each time, several
    microseconds per kernel launch; the raw accessor does not.)"""
    global _DEVICE_INDEX
    if _RAW_STREAM is None:
        return torch.cuda.current_stream().cuda_stream
    if _DEVICE_INDEX is None:
        _DEVICE_INDEX = torch.cuda.current_device()
    return _RAW_STREAM(_DEVICE_INDEX)


def _ptr(t) -> int:
    return 0 if t is None else t.data_ptr()


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise InvalidArgument(msg)


def _dev(*ts) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise InvalidArgument("kernel arguments must be CUDA tensors: the engine has no CPU path")


class SplitSum:
    """The result of a matrix product whose k range was cut into splits, not yet added up:
    float32 partial sums [splits, M, N] in scratch memory. Kernels that consume it (the residual
    add + norm, the q/k norm + RoPE + append) add the splits in order while they read, which saves
    a reduction kernel and a rounding; `materialize` adds them into a tensor for everyone else."""

    def __init__(self, partial: torch.Tensor, splits: int, M: int, N: int):
        self.partial, self.splits, self.M, self.N = partial, splits, M, N

    @property
    def stride(self) -> int:
        return self.M * self.N

    def materialize(self, out: torch.Tensor) -> torch.Tensor:
        p = self.partial[:self.splits * self.stride].view(self.splits, self.M, self.N)
        out.copy_(p.sum(dim=0) if self.splits > 1 else p[0])   # off the product path: toy parts and tests only
        return out


def embed(table: torch.Tensor, ids: torch.Tensor, out: torch.Tensor) -> None:
    """out[t] = float(table[ids[t]]); out is the float32 residual stream [T, D]. The table is [V, D], or the
    same in k-blocks, [ceil(D / 64), V, 64] (`pack_k_blocks`: what a tied output table is stored as)."""
    _dev(table, ids, out)
    T, D = out.shape
    packed = table.dim() == 3
    _need(table.is_contiguous() and ((not packed and table.dim() == 2 and table.shape[1] == D) or
                                     (packed and table.shape[2] == 64 and table.shape[0] == (D + 63) // 64)),
          "embed: table must be [V, D] or [ceil(D / 64), V, 64], contiguous")
    _need(ids.dtype == torch.int32 and ids.numel() == T and ids.is_contiguous(), "embed: ids must be int32 [T]")
    _need(out.dtype == torch.float32 and out.is_contiguous(), "embed: output must be float32 contiguous")
    V = table.shape[1] if packed else table.shape[0]
    call("tie_embed", dtype_code(table), table.data_ptr(), ids.data_ptr(), out.data_ptr(), T, D, V, V if packed else 0, _stream())


def pack_k_blocks(w: torch.Tensor) -> torch.Tensor:
    """[N, K] -> [ceil(K / 64), N, 64]: the rows' first 64 columns, then their next 64, and so on (zeros beyond K).
    The tensor-core products load a weight in boxes of 128 rows x 64 columns; stored like this a box is one piece
    of 16 KB instead of 128 pieces of 128 bytes a row apart, which is what the memory streams fastest."""
    N, K = w.shape
    kb = (K + 63) // 64
    if K % 64:
        w = torch.nn.functional.pad(w, (0, kb * 64 - K))
    return w.view(N, kb, 64).permute(1, 0, 2).contiguous()


def unpack_k_blocks(packed: torch.Tensor, K: int) -> torch.Tensor:
    """The inverse of pack_k_blocks: [ceil(K / 64), N, 64] -> [N, K] (a copy)."""
    kb, N, _ = packed.shape
    return packed.permute(1, 0, 2).reshape(N, kb * 64)[:, :K].contiguous()


def scatter_ids(tokens: torch.Tensor, dst: torch.Tensor, src: torch.Tensor, ids: torch.Tensor, n: int) -> None:
    """tokens[dst[i]] = ids[src[i]] for i < n (all int32): sampled ids of the step before become input tokens of
    this one without a trip to the host."""
    _dev(tokens, dst, src, ids)
    _need(all(t.dtype == torch.int32 and t.is_contiguous() for t in (tokens, dst, src, ids)) and
          0 <= n <= min(dst.numel(), src.numel()), "scatter_ids: int32 contiguous arrays, n within dst and src")
    call("tie_scatter_ids", tokens.data_ptr(), dst.data_ptr(), src.data_ptr(), ids.data_ptr(), n, _stream())


def add_rmsnorm(x: torch.Tensor, delta, weight: torch.Tensor, eps: float, out: torch.Tensor, rows=None) -> None:
    """x += delta (when given; float32, in place), out = rmsnorm(x) * weight in out's dtype.
    With `rows` (int32 [R]), out[i] comes from row rows[i] and x is left as it is. `delta` may
    be a SplitSum: its splits are added in order while they are read."""
    part = None
    if isinstance(delta, SplitSum):
        part, delta = delta, None
        _need(part.M == x.shape[0] and part.N == x.shape[-1], "add_rmsnorm: partial sums do not match x")
    _dev(x, delta, weight, out, rows)
    D = x.shape[-1]
    n = out.shape[0]
    _need(x.dtype == torch.float32 and x.is_contiguous(), "add_rmsnorm: x must be float32 contiguous")
    _need(weight.dtype == torch.float32 and weight.numel() == D, "add_rmsnorm: weight must be float32 [D]")
    _need(out.shape[-1] == D and out.is_contiguous(), "add_rmsnorm: out must be [n, D] contiguous")
    if delta is not None:
        _need(delta.dtype == out.dtype and delta.shape == x.shape and delta.is_contiguous(),
              "add_rmsnorm: delta must match x's shape and out's dtype")
    if rows is None:
        _need(n == x.shape[0], "add_rmsnorm: out must have x's rows")
    else:
        _need(rows.dtype == torch.int32 and rows.numel() == n, "add_rmsnorm: rows must be int32 [n]")
    call("tie_add_rmsnorm", dtype_code(out), x.data_ptr(), _ptr(delta), part.partial.data_ptr() if part else 0,
         part.stride if part else 0, part.splits if part else 0, _ptr(rows), weight.data_ptr(), float(eps), out.data_ptr(),
         n, D, _stream())


def rmsnorm_rows(x: torch.Tensor, weight: torch.Tensor, eps: float, out: torch.Tensor) -> None:
    """RMSNorm over the last axis of a 2-D view whose rows may be strided (last axis contiguous)."""
    _dev(x, weight, out)
    _need(x.dim() == 2 and out.shape == x.shape and x.dtype == out.dtype, "rmsnorm_rows: x and out must be 2-D alike")
    _need(x.stride(1) == 1 and out.stride(1) == 1, "rmsnorm_rows: last axis must be contiguous")
    _need(weight.dtype == torch.float32 and weight.numel() == x.shape[1], "rmsnorm_rows: weight must be float32 [size]")
    call("tie_rmsnorm_rows", dtype_code(x), x.data_ptr(), x.stride(0), weight.data_ptr(), float(eps), out.data_ptr(),
         out.stride(0), x.shape[1], x.shape[0], _stream())


def silu_mul(gate_up: torch.Tensor, out: torch.Tensor) -> None:
    """out[t, i] = silu(gate_up[t, i]) * gate_up[t, I + i]."""
    _dev(gate_up, out)
    T, I = out.shape
    _need(gate_up.shape == (T, 2 * I) and gate_up.is_contiguous() and out.is_contiguous() and
          gate_up.dtype == out.dtype, "silu_mul: gate_up must be [T, 2I] and out [T, I], same dtype, contiguous")
    call("tie_silu_mul", dtype_code(out), gate_up.data_ptr(), out.data_ptr(), T, I, _stream())


def rope(x: torch.Tensor, positions: torch.Tensor, inv_freq: torch.Tensor, heads: int, head_dim: int) -> None:
    """Rotate-half RoPE in place over the first 2*len(inv_freq) dims of each head of x [T, >= heads*head_dim]."""
    _dev(x, positions, inv_freq)
    _need(x.dim() == 2 and x.stride(1) == 1 and x.shape[1] >= heads * head_dim, "rope: x must be [T, heads*head_dim]")
    _need(positions.dtype == torch.int32 and positions.numel() == x.shape[0], "rope: positions must be int32 [T]")
    _need(inv_freq.dtype == torch.float32, "rope: inv_freq must be float32")
    call("tie_rope", dtype_code(x), x.data_ptr(), x.stride(0), positions.data_ptr(), inv_freq.data_ptr(), x.shape[0],
         heads, head_dim, 2 * inv_freq.numel(), _stream())


def _check_planes(k_cache, v_cache, kv_heads, head_dim):
    _need(k_cache.dim() == 4 and k_cache.shape == v_cache.shape and k_cache.is_contiguous() and v_cache.is_contiguous(),
          "cache planes must be [pages, kv_heads, page_size, head_dim] contiguous")
    _need(k_cache.shape[1] == kv_heads and k_cache.shape[3] == head_dim, "cache planes do not match the heads")
    _need(k_cache.numel() // head_dim < 2 ** 31, "cache plane too large for 32-bit row indices")


def kv_append(k: torch.Tensor, v: torch.Tensor, slots: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor) -> None:
    """k, v [T, kv_heads*head_dim] (rows may be strided) into the planes at slots[t]; slot < 0 writes nothing."""
    _dev(k, v, slots, k_cache, v_cache)
    kv_heads, page_size, head_dim = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3]
    _check_planes(k_cache, v_cache, kv_heads, head_dim)
    _need(k.shape == v.shape and k.shape[1] == kv_heads * head_dim and k.stride(1) == 1 and v.stride(1) == 1,
          "kv_append: k and v must be [T, kv_heads*head_dim]")
    _need(k.dtype == k_cache.dtype and v.dtype == k_cache.dtype, "kv_append: dtype differs from the cache's")
    _need(slots.dtype == torch.int32 and slots.numel() == k.shape[0], "kv_append: slots must be int32 [T]")
    call("tie_kv_append", dtype_code(k), k.data_ptr(), v.data_ptr(), k.stride(0), v.stride(0), slots.data_ptr(),
         k_cache.data_ptr(), v_cache.data_ptr(), k.shape[0], kv_heads, head_dim, page_size, _stream())


def qk_norm_rope_append(qkv: torch.Tensor, q_weight, k_weight, q_eps: float, k_eps: float, inv_freq,
                        positions: torch.Tensor, slots, k_cache, v_cache, q_heads: int, kv_heads: int,
                        head_dim: int, write_kv: bool = True, partial: SplitSum | None = None) -> None:
    """Per-head RMSNorm of q and k (weights may be None), RoPE (inv_freq may be None), q back in
    place, k and v into the cache planes. qkv is [T, (q_heads + 2 kv_heads) * head_dim]; with
    write_kv False it may hold q only and the planes are not touched. With `partial` the values
    are read from the split product's partial sums [splits, T, width] and only q is written to qkv."""
    _dev(qkv, q_weight, k_weight, inv_freq, positions, slots, k_cache, v_cache)
    T = qkv.shape[0]
    width = (q_heads + (2 * kv_heads if write_kv else 0)) * head_dim
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= width, "qk_norm_rope_append: qkv too narrow")
    _need(positions.dtype == torch.int32 and positions.numel() == T, "qk_norm_rope_append: positions must be int32 [T]")
    for w in (q_weight, k_weight):
        _need(w is None or (w.dtype == torch.float32 and w.numel() == head_dim),
              "qk_norm_rope_append: norm weights must be float32 [head_dim]")
    rot = 0
    if inv_freq is not None:
        _need(inv_freq.dtype == torch.float32, "qk_norm_rope_append: inv_freq must be float32")
        rot = 2 * inv_freq.numel()
    page_size = 1
    if write_kv:
        _check_planes(k_cache, v_cache, kv_heads, head_dim)
        _need(k_cache.dtype == qkv.dtype, "qk_norm_rope_append: dtype differs from the cache's")
        _need(slots.dtype == torch.int32 and slots.numel() == T, "qk_norm_rope_append: slots must be int32 [T]")
        page_size = k_cache.shape[2]
    if partial is not None:
        _need(partial.M == T and partial.N == width, "qk_norm_rope_append: partial sums do not match the rows")
    call("tie_qk_norm_rope_append", dtype_code(qkv), qkv.data_ptr(), qkv.stride(0),
         partial.partial.data_ptr() if partial else 0, partial.stride if partial else 0, partial.splits if partial else 0,
         partial.N if partial else 0, _ptr(q_weight), _ptr(k_weight),
         float(q_eps), float(k_eps), _ptr(inv_freq), rot, positions.data_ptr(), _ptr(slots) if write_kv else 0,
         _ptr(k_cache) if write_kv else 0, _ptr(v_cache) if write_kv else 0, T, q_heads, kv_heads, head_dim, page_size,
         1 if write_kv else 0, _stream())


def gemm_simt(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, N] = a[M, K] . w[N, K]^T on the CUDA cores with float accumulation (any sizes)."""
    _dev(a, w, out)
    _need(a.dim() == 2 and w.dim() == 2 and out.dim() == 2, "gemm: operands must be 2-D")
    M, K = a.shape
    N = w.shape[0]
    _need(w.shape[1] == K and out.shape == (M, N), f"gemm: shapes {tuple(a.shape)} x {tuple(w.shape)}^T -> {tuple(out.shape)}")
    _need(a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1, "gemm: last axes must be contiguous")
    _need(a.dtype == w.dtype, "gemm: a and w must have one dtype")
    call("tie_gemm_simt", dtype_code(a), dtype_code(out), a.data_ptr(), w.data_ptr(), out.data_ptr(), M, N, K,
         a.stride(0), w.stride(0), out.stride(0), _stream())


def _attn_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim):
    _check_planes(k_cache, v_cache, kv_heads, head_dim)
    _need(q.dim() == 2 and q.stride(1) == 1 and q.shape[1] >= q_heads * head_dim, "attention: q too narrow")
    _need(out.shape == (q.shape[0], q_heads * head_dim) and out.is_contiguous(), "attention: out must be [T, Hq*Dh]")
    _need(q.dtype == k_cache.dtype and out.dtype == q.dtype, "attention: q, cache and out must have one dtype")
    S = context_lens.numel()
    _need(query_start.dtype == torch.int32 and query_start.numel() == S + 1, "attention: query_start must be int32 [S+1]")
    _need(context_lens.dtype == torch.int32, "attention: context_lens must be int32 [S]")
    _need(block_tables.dtype == torch.int32 and block_tables.dim() == 2 and block_tables.shape[0] == S and
          block_tables.is_contiguous(), "attention: block_tables must be int32 [S, max_blocks]")
    return S


def attention_rows(q, k_cache, v_cache, out, seq_of_row, query_start, context_lens, block_tables, q_heads, kv_heads,
                   head_dim, scale: float, window: int = 0) -> None:
    """Causal attention of every row of the step over the paged cache (CUDA cores)."""
    _dev(q, k_cache, v_cache, out, seq_of_row, query_start, context_lens, block_tables)
    S = _attn_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim)
    _need(seq_of_row.dtype == torch.int32 and seq_of_row.numel() == q.shape[0], "attention: seq_of_row must be int32 [T]")
    call("tie_attention_rows", dtype_code(q), q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
         out.data_ptr(), seq_of_row.data_ptr(), query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(),
         block_tables.shape[1], q.shape[0], S, q_heads, kv_heads, head_dim, k_cache.shape[2], int(window), float(scale),
         _stream())


def attention_split_scratch_floats(n_list: int, q_heads: int, head_dim: int, max_splits: int) -> int:
    return n_list * q_heads * max_splits * (head_dim + 2)


def attention_split(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim,
                    scale: float, seq_list, n_list: int, split_keys: int, max_splits: int, scratch,
                    window: int = 0) -> None:
    """Attention of sequences that bring one token each, their keys cut into splits of `split_keys`."""
    _dev(q, k_cache, v_cache, out, query_start, context_lens, block_tables, seq_list, scratch)
    S = _attn_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim)
    _need(seq_list.dtype == torch.int32 and seq_list.numel() >= n_list, "attention: seq_list must be int32 [n_list]")
    _need(scratch.dtype == torch.float32 and
          scratch.numel() >= attention_split_scratch_floats(n_list, q_heads, head_dim, max_splits),
          "attention: scratch too small")
    call("tie_attention_split", dtype_code(q), q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
         out.data_ptr(), query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1],
         S, q_heads, kv_heads, head_dim, k_cache.shape[2], int(window), float(scale), seq_list.data_ptr(), n_list,
         split_keys, max_splits, scratch.data_ptr(), _stream())


def attention_tc_takes(q: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int) -> bool:
    """Whether the tensor-core attention kernels take these operands (else the CUDA-core ones do)."""
    return (q.dtype == torch.bfloat16 and head_dim in (64, 128, 256) and q_heads // kv_heads <= 16 and
            q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0)


def attention_prompt_tc(q, k_cache, v_cache, out, query_start, context_lens, block_tables, n_seqs: int, max_queries: int,
                        q_heads, kv_heads, head_dim, scale: float, window: int = 0) -> None:
    """Tensor-core attention of the first n_seqs sequences of the step (each brings several tokens;
    their rows come first); max_queries is the most tokens one of them brings."""
    _dev(q, k_cache, v_cache, out, query_start, context_lens, block_tables)
    _attn_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim)
    call("tie_attention_prompt_tc", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
         query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], n_seqs,
         max_queries, q_heads, kv_heads, head_dim, k_cache.shape[2], int(window), float(scale), _stream())


def attention_decode_tc(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim,
                        scale: float, seq_list, n_list: int, split_keys: int, max_splits: int, scratch,
                        window: int = 0) -> None:
    """Tensor-core attention of sequences that bring one token each: split kernel, then the merge."""
    _dev(q, k_cache, v_cache, out, query_start, context_lens, block_tables, seq_list, scratch)
    _attn_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim)
    _need(seq_list.dtype == torch.int32 and seq_list.numel() >= n_list, "attention: seq_list must be int32 [n_list]")
    _need(scratch.dtype == torch.float32 and
          scratch.numel() >= attention_split_scratch_floats(n_list, q_heads, head_dim, max_splits),
          "attention: scratch too small")
    call("tie_attention_decode_tc", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
         query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], q_heads, kv_heads,
         head_dim, k_cache.shape[2], int(window), float(scale), seq_list.data_ptr(), n_list, split_keys, max_splits,
         scratch.data_ptr(), _stream())
    call("tie_attention_merge", dtype_code(out), out.data_ptr(), query_start.data_ptr(), context_lens.data_ptr(), q_heads,
         head_dim, int(window), seq_list.data_ptr(), n_list, split_keys, max_splits, scratch.data_ptr(), _stream())


def attention_decode_tma_takes(q: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the TMA-fed attention kernels (decode and prompt) take these operands."""
    return attention_tc_takes(q, q_heads, kv_heads, head_dim) and page_size >= 8 and page_size & (page_size - 1) == 0


def attention_prompt_tma(q, k_cache, v_cache, out, query_start, context_lens, block_tables, n_seqs: int, max_queries: int,
                         q_heads, kv_heads, head_dim, scale: float, window: int = 0, exact_weights: bool = False) -> None:
    """As attention_prompt_tc, keys and values fed by TMA (pages that are powers of two from 8 up). `exact_weights`:
    the float softmax weights enter the value product as two bfloat16 terms, hi + lo (16 bits of mantissa), for
    models whose softmax weights are to stay 32-bit; twice the MMAs of that product."""
    _dev(q, k_cache, v_cache, out, query_start, context_lens, block_tables)
    _attn_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim)
    call("tie_attention_prompt_tma_exact" if exact_weights else "tie_attention_prompt_tma", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
         query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], n_seqs,
         max_queries, q_heads, kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0], int(window), float(scale), _stream())


_NO_UMMA_ATTENTION = os.environ.get("TIE_NO_UMMA_ATTENTION") == "1"
UMMA_MIN_ROWS = 128     # rows (queries x heads of a group) from which the tcgen05 prompt kernel pays


def attention_prompt_umma_takes(q: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int, page_size: int,
                                max_queries: int) -> bool:
    """Whether the tcgen05 prompt kernel takes these operands and the portions are long enough for its
    256-row tiles."""
    return (attention_decode_tma_takes(q, q_heads, kv_heads, head_dim, page_size) and head_dim in (64, 128)
            and max_queries * (q_heads // kv_heads) >= UMMA_MIN_ROWS and not _NO_UMMA_ATTENTION)


def attention_prompt_umma(q, k_cache, v_cache, out, query_start, context_lens, block_tables, n_seqs: int, max_queries: int,
                          q_heads, kv_heads, head_dim, scale: float, window: int = 0) -> None:
    """As attention_prompt_tma with both products on tcgen05 and the accumulators in tensor memory
    (head sizes 64 and 128)."""
    _dev(q, k_cache, v_cache, out, query_start, context_lens, block_tables)
    _attn_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim)
    _need(out.is_contiguous(), "attention: out must be contiguous")
    call("tie_attention_prompt_umma", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
         query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], n_seqs,
         max_queries, q_heads, kv_heads, head_dim, k_cache.shape[2], k_cache.shape[0], int(window), float(scale), _stream())


CLUSTER_SPLITS = (2, 4, 8, 16)      # how many splits the decode attention merges as one thread-block cluster


def attention_decode_tma(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim,
                         scale: float, seq_list, n_list: int, split_keys: int, max_splits: int, scratch, counters,
                         window: int = 0, cluster: bool = False, exact_weights: bool = False) -> None:
    """Attention of sequences that bring one token each, keys and values fed by TMA, splits merged by
    the last CTA to finish. `exact_weights` as in `attention_prompt_tma`. `counters` (int32 [>= n_list * kv_heads]) must be zero; it is left zero.
    `cluster` (with max_splits in CLUSTER_SPLITS): the splits of a sequence and kv head run as one thread-block
    cluster and merge through shared memory, which is faster where all the launch's CTAs are resident at once.
    `seq_list`: int32 [n_list], or an int: the first of n_list sequences in a row (the kernel then has one load
    less to wait for before it can ask for keys)."""
    first = seq_list if isinstance(seq_list, int) else 0
    seq_list = None if isinstance(seq_list, int) else seq_list
    _dev(q, k_cache, v_cache, out, query_start, context_lens, block_tables, seq_list, scratch, counters)
    S = _attn_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim)
    _need((seq_list is None and 0 <= first and first + n_list <= S) or
          (seq_list is not None and seq_list.dtype == torch.int32 and seq_list.numel() >= n_list),
          "attention: seq_list must be int32 [n_list], or the first of n_list sequences in a row")
    _need(scratch.dtype == torch.float32 and
          scratch.numel() >= attention_split_scratch_floats(n_list, q_heads, head_dim, max_splits),
          "attention: scratch too small")
    _need(counters.dtype == torch.int32 and counters.numel() >= n_list * kv_heads, "attention: counters too small")
    call("tie_attention_decode_tma_exact" if exact_weights else "tie_attention_decode_tma", q.data_ptr(), q.stride(0),
         k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
         query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], q_heads, kv_heads,
         head_dim, k_cache.shape[2], k_cache.shape[0], int(window), float(scale), _ptr(seq_list), first, n_list, split_keys,
         max_splits, scratch.data_ptr(), counters.data_ptr(), 1 if cluster else 0, _stream())


def attention_decode_prep_takes(qkv: torch.Tensor, q_heads: int, kv_heads: int, head_dim: int, page_size: int, inv_freq) -> bool:
    """Whether the decode attention that prepares its own heads takes these operands: what the TMA-fed kernel takes,
    and a rotation (if any) over the whole head."""
    return (attention_decode_tma_takes(qkv, q_heads, kv_heads, head_dim, page_size)
            and (inv_freq is None or 2 * inv_freq.numel() == head_dim))


def attention_decode_prep(qkv, q_weight, k_weight, q_eps: float, k_eps: float, inv_freq, positions, k_cache, v_cache, out,
                          query_start, context_lens, block_tables, q_heads, kv_heads, head_dim, scale: float, seq_list,
                          n_list: int, split_keys: int, max_splits: int, scratch, counters, window: int = 0,
                          append: bool = True, partial: SplitSum | None = None, cluster: bool = False) -> None:
    """`attention_decode_tma` for a step in which every sequence brings one token, straight from the q/k/v product's
    output: qkv [T, (q_heads + 2 kv_heads) * head_dim] (or q only, with `append` False), or the product's partial sums.
    The kernel does what `qk_norm_rope_append` does to the group's query heads and, with `append`, to the newest
    key and value, which it stores in the cache planes and uses; qkv itself is left as it is."""
    first = seq_list if isinstance(seq_list, int) else 0
    seq_list = None if isinstance(seq_list, int) else seq_list
    _dev(qkv, q_weight, k_weight, inv_freq, positions, k_cache, v_cache, out, query_start, context_lens, block_tables,
         seq_list, scratch, counters)
    T = qkv.shape[0]
    width = (q_heads + (2 * kv_heads if append else 0)) * head_dim
    _need(qkv.dim() == 2 and qkv.stride(1) == 1 and qkv.shape[1] >= width and qkv.dtype == torch.bfloat16,
          "attention_decode_prep: qkv must be bfloat16 rows of q (and k, v)")
    _need(out.shape == (T, q_heads * head_dim) and out.is_contiguous() and out.dtype == torch.bfloat16,
          "attention_decode_prep: out must be contiguous bfloat16 [T, q_heads * head_dim]")
    _check_planes(k_cache, v_cache, kv_heads, head_dim)
    _need(k_cache.dtype == torch.bfloat16, "attention_decode_prep: the cache must be bfloat16")
    _need(positions.dtype == torch.int32 and positions.numel() == T, "attention_decode_prep: positions must be int32 [T]")
    for w in (q_weight, k_weight):
        _need(w is None or (w.dtype == torch.float32 and w.numel() == head_dim),
              "attention_decode_prep: norm weights must be float32 [head_dim]")
    _need(inv_freq is None or (inv_freq.dtype == torch.float32 and 2 * inv_freq.numel() == head_dim),
          "attention_decode_prep: the rotation must cover the whole head")
    _need(query_start.dtype == torch.int32 and context_lens.dtype == torch.int32 and block_tables.dtype == torch.int32
          and block_tables.dim() == 2 and block_tables.stride(1) == 1, "attention: index tensors must be int32")
    _need((seq_list is None and 0 <= first and first + n_list <= context_lens.numel()) or
          (seq_list is not None and seq_list.dtype == torch.int32 and seq_list.numel() >= n_list),
          "attention: seq_list must be int32 [n_list], or the first of n_list sequences in a row")
    _need(scratch.dtype == torch.float32 and
          scratch.numel() >= attention_split_scratch_floats(n_list, q_heads, head_dim, max_splits),
          "attention: scratch too small")
    _need(counters.dtype == torch.int32 and counters.numel() >= n_list * kv_heads, "attention: counters too small")
    if partial is not None:
        _need(partial.M == T and partial.N == width, "attention_decode_prep: partial sums do not match the rows")
    call("tie_attention_decode_prep", qkv.data_ptr(), qkv.stride(0), partial.partial.data_ptr() if partial else 0,
         partial.stride if partial else 0, partial.splits if partial else 0, partial.N if partial else 0,
         _ptr(q_weight), _ptr(k_weight), float(q_eps), float(k_eps), _ptr(inv_freq), positions.data_ptr(),
         1 if append else 0, k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), query_start.data_ptr(),
         context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], q_heads, kv_heads, head_dim,
         k_cache.shape[2], k_cache.shape[0], int(window), float(scale), _ptr(seq_list), first, n_list, split_keys,
         max_splits, scratch.data_ptr(), counters.data_ptr(), 1 if cluster else 0, _stream())


def sample(logits: torch.Tensor, out: torch.Tensor, inv_temperature=None, seeds=None, counters=None, top_k=None,
           top_p=None, one_cta: bool = False) -> None:
    """out[r] = first maximum of row r (inv_temperature None or 0), or a draw from softmax(logits * inv_temperature)
    with the Philox uniform of (seeds[r], counters[r]). With top_k (int32) and top_p (float32) the rows whose
    top_k is in (0, vocab) or whose top_p is below 1 draw from the candidates those keep, most likely first
    (`one_cta`: with the kernel that serves the largest vocabularies, whatever the size; for tests)."""
    _dev(logits, out, inv_temperature, seeds, counters, top_k, top_p)
    R, V = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "sample: logits must be float32 rows")
    _need(out.dtype == torch.int32 and out.numel() >= R, "sample: out must be int32 [R]")
    if inv_temperature is not None:
        _need(inv_temperature.dtype == torch.float32 and seeds.dtype == torch.int64 and counters.dtype == torch.int64,
              "sample: inv_temperature float32, seeds and counters int64")
    call("tie_sample", logits.data_ptr(), logits.stride(0), R, V, _ptr(inv_temperature), _ptr(seeds), _ptr(counters),
         out.data_ptr(), _stream())
    if top_k is not None or top_p is not None:
        _need(inv_temperature is not None and top_k is not None and top_p is not None,
              "sample: top_k and top_p come together, with temperatures")
        _need(top_k.dtype == torch.int32 and top_p.dtype == torch.float32 and top_k.numel() >= R and top_p.numel() >= R,
              "sample: top_k int32 [R], top_p float32 [R]")
        call("tie_sample_filtered", logits.data_ptr(), logits.stride(0), R, V, inv_temperature.data_ptr(), top_k.data_ptr(),
             top_p.data_ptr(), seeds.data_ptr(), counters.data_ptr(), out.data_ptr(), 1 if one_cta else 0, _stream())


def gemm(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, partial_scratch=None):
    """The engine's matrix product: picks the kernel for the dtype and the sizes. With
    `partial_scratch` (a callable numel -> float32 buffer) a product whose k range is split may
    come back as a SplitSum (then `out` is untouched); else returns `out`.

    `w` is taken for a weight: the tensor-core kernels start fetching it before the kernel ahead of them
    in the stream has finished, so it must not be something that kernel writes."""
    from . import gemm_select
    return gemm_select.gemm(a, w, out, partial_scratch)


def bound_gemm(w: torch.Tensor, silu: bool = False, split_many: bool = True, pack: bool = True):
    """A matrix product bound to one weight (gemm_select.BoundGemm): checked once, called every step.
    `split_many` False: above 128 tokens k is never split (the consumer wants the finished product). With `pack`
    a weight that the tensor-core kernels take is stored in k-blocks (pack_k_blocks) from here on: the product
    keeps that copy (`.w`) and the caller lets go of its own. `.rows(a, b)` is the product with rows a..b-1 of
    the same weight, without a copy."""
    from . import gemm_select
    return gemm_select.BoundGemm(w, silu, split_many, pack)


def partial_capacity(max_rows: int, N: int, K: int, split_many: bool = True) -> int:
    """The largest scratch (floats) a split product of up to max_rows tokens with [N, K] weights asks for."""
    from . import gemm_select
    return gemm_select.partial_capacity(int(max_rows), int(N), int(K), bool(split_many))


def gemm_silu(a: torch.Tensor, w_blocks: torch.Tensor, out: torch.Tensor) -> None:
    """out[M, I] = silu(a . gate^T) * (a . up^T) in one tensor-core product; w_blocks [2I, K] holds
    blocks of 16 gate rows followed by their 16 up rows (interleave_gate_up)."""
    from . import gemm_select
    gemm_select.gemm_silu(a, w_blocks, out)


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """[I, K], [I, K] -> [2I, K]: 16 gate rows, their 16 up rows, the next 16 gate rows, ... (I % 16 == 0)."""
    I, K = gate.shape
    return torch.stack([gate.view(I // 16, 16, K), up.view(I // 16, 16, K)], dim=1).reshape(2 * I, K).contiguous()


# -- layers that norm a sublayer's output before adding it, gated units, scaled logits (csrc/layer_glue.cu)

class NormedDelta:
    """A sublayer's output that is still to pass a norm of its own and a factor before it joins the residual
    stream: x += mult * ((y * inv_rms(y)) * weight), y = delta (+ bias). `delta` is a tensor [T, D] in the
    compute dtype or a SplitSum; `weight` float32 [D]; `bias` float32 [D] or None."""

    def __init__(self, delta, weight: torch.Tensor, eps: float, mult: float, bias=None):
        self.delta, self.weight, self.eps, self.mult, self.bias = delta, weight, float(eps), float(mult), bias


def add_normed_rmsnorm(x: torch.Tensor, pending: NormedDelta, weight: torch.Tensor, eps: float, out: torch.Tensor,
                       rows=None) -> None:
    """x += mult * norm_b(delta + bias) (float32, in place), out = rmsnorm(x) * weight in out's dtype. With `rows`
    (int32 [R]) out[i] comes from row rows[i] and x is left as it is."""
    part, delta = None, pending.delta
    if isinstance(delta, SplitSum):
        part, delta = delta, None
        _need(part.M == x.shape[0] and part.N == x.shape[-1], "add_normed_rmsnorm: partial sums do not match x")
    _dev(x, delta, weight, out, rows, pending.weight, pending.bias)
    D, n = x.shape[-1], out.shape[0]
    _need(x.dtype == torch.float32 and x.is_contiguous(), "add_normed_rmsnorm: x must be float32 contiguous")
    for w in (weight, pending.weight, pending.bias):
        _need(w is None or (w.dtype == torch.float32 and w.numel() == D), "add_normed_rmsnorm: weights and bias must be float32 [D]")
    _need(out.shape[-1] == D and out.is_contiguous(), "add_normed_rmsnorm: out must be [n, D] contiguous")
    if delta is not None:
        _need(delta.dtype == out.dtype and delta.shape == x.shape and delta.is_contiguous(),
              "add_normed_rmsnorm: delta must match x's shape and out's dtype")
    if rows is None:
        _need(n == x.shape[0], "add_normed_rmsnorm: out must have x's rows")
    else:
        _need(rows.dtype == torch.int32 and rows.numel() == n, "add_normed_rmsnorm: rows must be int32 [n]")
    call("tie_add_normed_rmsnorm", dtype_code(out), x.data_ptr(), _ptr(delta), part.partial.data_ptr() if part else 0,
         part.stride if part else 0, part.splits if part else 0, _ptr(pending.bias), pending.weight.data_ptr(), pending.eps,
         pending.mult, _ptr(rows), weight.data_ptr(), float(eps), out.data_ptr(), n, D, _stream())


def glu_clamped(gate_up: torch.Tensor, out: torch.Tensor, limit: float, slope: float, up_shift: float) -> None:
    """out[t, i] = g sigmoid(slope g) (u + up_shift), g = min(gate_up[t, i], limit), u = clamp(gate_up[t, I + i], -limit, limit)."""
    _dev(gate_up, out)
    T, I = out.shape
    _need(gate_up.shape == (T, 2 * I) and gate_up.is_contiguous() and out.is_contiguous() and gate_up.dtype == out.dtype,
          "glu_clamped: gate_up must be [T, 2I] and out [T, I], same dtype, contiguous")
    call("tie_glu_clamped", dtype_code(out), gate_up.data_ptr(), out.data_ptr(), T, I, float(limit), float(slope),
         float(up_shift), _stream())


def sigmoid_gate_mul(y: torch.Tensor, gate: torch.Tensor) -> None:
    """y *= sigmoid(gate), in place; both [T, W] with contiguous last axes (rows may be strided)."""
    _dev(y, gate)
    _need(y.dim() == 2 and y.shape == gate.shape and y.dtype == gate.dtype and y.stride(1) == 1 and gate.stride(1) == 1,
          "sigmoid_gate_mul: y and gate must be [T, W] alike")
    call("tie_sigmoid_gate_mul", dtype_code(y), y.data_ptr(), y.stride(0), gate.data_ptr(), gate.stride(0), y.shape[0],
         y.shape[1], _stream())


def scale_rows(x: torch.Tensor, c: float) -> None:
    """x *= c for float32 rows, in place."""
    _dev(x)
    _need(x.dim() == 2 and x.dtype == torch.float32 and x.stride(1) == 1, "scale_rows: x must be float32 rows")
    call("tie_scale_rows", x.data_ptr(), x.stride(0), x.shape[0], x.shape[1], float(c), _stream())


# -- attention with an RMS norm over the whole projection, biases, blended values, keys and values of two sizes

def _check_kv_planes(k_cache, v_cache, kv_heads, head_dim, v_dim):
    _need(k_cache.dim() == 4 and v_cache.dim() == 4 and k_cache.is_contiguous() and v_cache.is_contiguous() and
          k_cache.shape[:3] == v_cache.shape[:3] and k_cache.dtype == v_cache.dtype,
          "cache planes must be [pages, kv_heads, page_size, size] contiguous, alike but for the size")
    _need(k_cache.shape[1] == kv_heads and k_cache.shape[3] == head_dim and v_cache.shape[3] == v_dim,
          "cache planes do not match the heads")
    _need(max(k_cache.numel() // head_dim, v_cache.numel() // v_cache.shape[3]) < 2 ** 31, "cache plane too large for 32-bit row indices")


def qkv_span_prep(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, bq, bk, bv, wq, wk, eps: float, inv_freq,
                  positions: torch.Tensor, slots, k_cache, v_cache, q_heads: int, kv_heads: int, head_dim: int, v_dim: int,
                  mix_mode: int = 0, v_first=None, mix_weight=None, write_kv: bool = True) -> None:
    """proj [T, >= ...] holds the q, k and v projections of every token at columns q_off, k_off, v_off. q gets its
    bias, the RMS norm over all of its heads at once (weights wq, float32 [q_heads * head_dim]) and the rotation of
    the first 2 * len(inv_freq) dimensions of each head, and is written back in place; k likewise into the key
    plane; v gets its bias, is kept as `v_first` (mix_mode 1) or blended with it, (1 - w) v + w v_first (mix_mode 2,
    `mix_weight` a float32 device scalar), and goes into the value plane."""
    _dev(proj, bq, bk, bv, wq, wk, inv_freq, positions, slots, k_cache, v_cache, v_first, mix_weight)
    T = proj.shape[0]
    nq, nk, nv = q_heads * head_dim, kv_heads * head_dim, kv_heads * v_dim
    _need(proj.dim() == 2 and proj.stride(1) == 1 and q_off + nq <= proj.shape[1], "qkv_span_prep: q outside the projection")
    _need(positions.dtype == torch.int32 and positions.numel() == T, "qkv_span_prep: positions must be int32 [T]")
    for t, n in ((bq, nq), (bk, nk), (bv, nv), (wq, nq), (wk, nk)):
        _need(t is None or (t.dtype == torch.float32 and t.numel() == n), "qkv_span_prep: biases and norm weights must be float32 of the projection's size")
    _need(inv_freq is None or inv_freq.dtype == torch.float32, "qkv_span_prep: inv_freq must be float32")
    page = 1
    if write_kv:
        _need(max(k_off + nk, v_off + nv) <= proj.shape[1], "qkv_span_prep: k or v outside the projection")
        _need(v_cache.dim() == 4 and v_cache.shape[3] >= v_dim, "qkv_span_prep: value plane narrower than a value head")
        _check_kv_planes(k_cache, v_cache, kv_heads, head_dim, v_cache.shape[3])
        _need(k_cache.dtype == proj.dtype, "qkv_span_prep: dtype differs from the cache's")
        _need(slots.dtype == torch.int32 and slots.numel() == T, "qkv_span_prep: slots must be int32 [T]")
        page = k_cache.shape[2]
        if mix_mode:
            _need(v_first is not None and v_first.dtype == torch.float32 and v_first.is_contiguous() and
                  v_first.shape == (T, nv), "qkv_span_prep: v_first must be float32 [T, kv_heads * v_dim]")
            _need(mix_mode == 1 or (mix_weight is not None and mix_weight.dtype == torch.float32 and mix_weight.numel() == 1),
                  "qkv_span_prep: the blend's weight must be a float32 scalar on the device")
    call("tie_qkv_span_prep", dtype_code(proj), proj.data_ptr(), proj.stride(0), q_off, k_off, v_off, _ptr(bq), _ptr(bk), _ptr(bv),
         _ptr(wq), _ptr(wk), float(eps), _ptr(inv_freq), 2 * inv_freq.numel() if inv_freq is not None else 0,
         positions.data_ptr(), _ptr(slots) if write_kv else 0, _ptr(k_cache) if write_kv else 0,
         _ptr(v_cache) if write_kv else 0, T, q_heads, kv_heads, head_dim, v_dim, v_cache.shape[3] if write_kv else v_dim, page,
         int(mix_mode) if write_kv else 0,
         _ptr(v_first), _ptr(mix_weight), _stream())


def _attn_common_dv(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim, v_dim,
                    values_in_keys: bool = False):
    if values_in_keys:
        _need(v_cache is k_cache or v_cache.data_ptr() == k_cache.data_ptr(), "attention: values in keys take the key plane twice")
        _need(v_dim <= head_dim, "attention: a value inside its key cannot be longer than the key")
        _check_kv_planes(k_cache, k_cache, kv_heads, head_dim, head_dim)
    else:
        _check_kv_planes(k_cache, v_cache, kv_heads, head_dim, v_dim)
    _need(q.dim() == 2 and q.stride(1) == 1 and q.shape[1] >= q_heads * head_dim, "attention: q too narrow")
    _need(out.shape == (q.shape[0], q_heads * v_dim) and out.is_contiguous(), "attention: out must be [T, Hq*Dv]")
    _need(q.dtype == k_cache.dtype and out.dtype == q.dtype, "attention: q, cache and out must have one dtype")
    S = context_lens.numel()
    _need(query_start.dtype == torch.int32 and query_start.numel() == S + 1, "attention: query_start must be int32 [S+1]")
    _need(context_lens.dtype == torch.int32, "attention: context_lens must be int32 [S]")
    _need(block_tables.dtype == torch.int32 and block_tables.dim() == 2 and block_tables.shape[0] == S and
          block_tables.is_contiguous(), "attention: block_tables must be int32 [S, max_blocks]")
    return S


def attention_rows_dv(q, k_cache, v_cache, out, seq_of_row, query_start, context_lens, block_tables, q_heads, kv_heads,
                      head_dim, v_dim, scale: float, window: int = 0, values_in_keys: bool = False) -> None:
    """`attention_rows` for keys of head_dim and values of v_dim (out [T, q_heads * v_dim]). `values_in_keys`: there
    is no value plane; a value is the first v_dim elements of its key (pass the key plane as `v_cache`)."""
    _dev(q, k_cache, v_cache, out, seq_of_row, query_start, context_lens, block_tables)
    S = _attn_common_dv(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim, v_dim,
                        values_in_keys)
    _need(seq_of_row.dtype == torch.int32 and seq_of_row.numel() == q.shape[0], "attention: seq_of_row must be int32 [T]")
    call("tie_attention_rows_dv", dtype_code(q), q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
         out.data_ptr(), seq_of_row.data_ptr(), query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(),
         block_tables.shape[1], q.shape[0], S, q_heads, kv_heads, head_dim, v_dim, k_cache.shape[2], int(window), float(scale),
         head_dim if values_in_keys else 0, _stream())


def attention_split_dv(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim, v_dim,
                       scale: float, seq_list, n_list: int, split_keys: int, max_splits: int, scratch, window: int = 0,
                       values_in_keys: bool = False) -> None:
    """`attention_split` for keys of head_dim and values of v_dim; scratch holds
    attention_split_scratch_floats(n_list, q_heads, v_dim, max_splits) floats. `values_in_keys` as in `attention_rows_dv`."""
    _dev(q, k_cache, v_cache, out, query_start, context_lens, block_tables, seq_list, scratch)
    S = _attn_common_dv(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, kv_heads, head_dim, v_dim,
                        values_in_keys)
    _need(seq_list.dtype == torch.int32 and seq_list.numel() >= n_list, "attention: seq_list must be int32 [n_list]")
    _need(scratch.dtype == torch.float32 and
          scratch.numel() >= attention_split_scratch_floats(n_list, q_heads, v_dim, max_splits), "attention: scratch too small")
    call("tie_attention_split_dv", dtype_code(q), q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(),
         out.data_ptr(), query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1],
         S, q_heads, kv_heads, head_dim, v_dim, k_cache.shape[2], int(window), float(scale), seq_list.data_ptr(), n_list,
         split_keys, max_splits, scratch.data_ptr(), head_dim if values_in_keys else 0, _stream())


# -- the gated delta rule with a decay per key channel (csrc/delta_rule.cu)

def delta_prep(proj, q_off: int, k_off: int, v_off: int, b_off: int, conv_w, state, conv_state_off: int, seq_of_row,
               query_start, state_slots, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, unit_eps: float,
               q_scale: float, qn, kn, vn, beta, decay, dt_bias, a_log) -> None:
    """Short causal convolution + SiLU of the q, k, v columns of `proj`, unit norm of q and k per head (q times
    q_scale), sigmoid of the beta columns. `state` [slots, floats] holds, from conv_state_off on, each sequence's
    last taps - 1 convolution inputs. Outputs are float32: qn, kn [T, kv_heads * dim], vn [T, heads * vdim], beta [T, heads].
    `decay` float32 [T, >= heads * dim] (rows may be strided) comes in as the raw decay projection a and leaves as
    exp(-exp(a_log[h]) softplus(a + dt_bias)) per head and key channel."""
    _dev(proj, conv_w, state, seq_of_row, query_start, state_slots, qn, kn, vn, beta, decay, dt_bias, a_log)
    T = proj.shape[0]
    nqk, nv = kv_heads * dim, heads * vdim
    _need(proj.dim() == 2 and proj.stride(1) == 1 and max(q_off + nqk, k_off + nqk, v_off + nv, b_off + heads) <= proj.shape[1],
          "delta_prep: columns outside the projection")
    _need(conv_w.dtype == torch.float32 and conv_w.is_contiguous() and conv_w.shape == (2 * nqk + nv, taps),
          "delta_prep: convolution weights must be float32 [channels, taps]")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1 and
          conv_state_off + (taps - 1) * (2 * nqk + nv) <= state.shape[1], "delta_prep: state rows too short")
    for t, n in ((qn, nqk), (kn, nqk), (vn, nv), (beta, heads)):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.shape == (T, n), "delta_prep: outputs must be float32 [T, n]")
    for t in (seq_of_row, query_start, state_slots):
        _need(t.dtype == torch.int32, "delta_prep: index tensors must be int32")
    _need(decay.dtype == torch.float32 and decay.dim() == 2 and decay.stride(1) == 1 and decay.shape[0] == T and
          decay.shape[1] >= heads * dim, "delta_prep: decay must be float32 [T, >= heads * dim]")
    _need(dt_bias.dtype == torch.float32 and dt_bias.numel() == heads * dim and a_log.dtype == torch.float32 and
          a_log.numel() == heads, "delta_prep: dt_bias float32 [heads * dim], a_log float32 [heads]")
    call("tie_delta_prep", dtype_code(proj), proj.data_ptr(), proj.stride(0), q_off, k_off, v_off, b_off, conv_w.data_ptr(),
         state.data_ptr(), state.stride(0), conv_state_off, seq_of_row.data_ptr(), query_start.data_ptr(),
         state_slots.data_ptr(), T, heads, kv_heads, dim, vdim, taps, float(unit_eps), float(q_scale), qn.data_ptr(),
         kn.data_ptr(), vn.data_ptr(), beta.data_ptr(), decay.data_ptr(), decay.stride(0), dt_bias.data_ptr(), a_log.data_ptr(),
         _stream())


def delta_rule(qn, kn, vn, beta, decay, state, conv_state_off: int, proj, q_off: int, k_off: int, v_off: int,
               query_start, state_slots, seqs: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, out,
               plain: bool = False, decay_per_head: bool = False) -> None:
    """The recurrence over each sequence's tokens of the step: per head S <- decay S; u = beta (v - S^T k);
    S <- S + k u^T; o = S^T q, with `decay` float32 [T, >= heads * dim] per head and key channel (`delta_prep`).
    S [heads, dim, vdim] sits at the start of the sequence's row of `state` and is updated; so are the convolution's
    last inputs (from the q, k, v columns of `proj`). out float32 [T, heads * vdim].
    `plain`: no correction, u = beta v (beta None: u = v), which is the recurrence of gated linear attention and of
    state-space layers, S <- diag(decay) S + k u^T. `decay_per_head`: decay is float32 [T, >= heads], one factor for
    all key channels of a head."""
    _dev(qn, kn, vn, beta, decay, state, proj, query_start, state_slots, out)
    T = proj.shape[0]
    _need(beta is not None or plain, "delta_rule: the delta rule needs beta")
    _need(decay.dtype == torch.float32 and decay.dim() == 2 and decay.stride(1) == 1 and decay.shape[0] == T and
          decay.shape[1] >= (heads if decay_per_head else heads * dim), "delta_rule: decay must be float32 [T, >= heads * dim]")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (T, heads * vdim), "delta_rule: out must be float32 [T, heads * vdim]")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1 and conv_state_off >= heads * dim * vdim,
          "delta_rule: state rows too short")
    _need(query_start.numel() >= seqs + 1 and state_slots.numel() >= seqs, "delta_rule: index tensors too short")
    call("tie_delta_rule", dtype_code(proj), qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), _ptr(beta), decay.data_ptr(),
         decay.stride(0), state.data_ptr(), state.stride(0), conv_state_off, proj.data_ptr(), proj.stride(0), q_off, k_off, v_off,
         query_start.data_ptr(), state_slots.data_ptr(), seqs, heads, kv_heads, dim, vdim, taps, out.data_ptr(),
         1 if plain else 0, 1 if decay_per_head else 0, _stream())


def delta_out(o, gate, weight, eps: float, out, heads: int, vdim: int) -> None:
    """out[t, h] = (o[t, h] / rms(o[t, h])) * weight * sigmoid(gate[t, h]) per head of vdim; o, gate float32, out in
    the compute dtype."""
    _dev(o, gate, weight, out)
    T = o.shape[0]
    _need(o.dtype == torch.float32 and o.is_contiguous() and o.shape == (T, heads * vdim), "delta_out: o must be float32 [T, heads * vdim]")
    _need(gate.dtype == torch.float32 and gate.dim() == 2 and gate.stride(1) == 1 and gate.shape == o.shape,
          "delta_out: gate must be float32 [T, heads * vdim]")
    _need(weight.dtype == torch.float32 and weight.numel() == vdim, "delta_out: weight must be float32 [vdim]")
    _need(out.is_contiguous() and out.shape == o.shape, "delta_out: out must be [T, heads * vdim] contiguous")
    call("tie_delta_out", dtype_code(out), o.data_ptr(), gate.data_ptr(), gate.stride(0), weight.data_ptr(), float(eps),
         out.data_ptr(), T, heads, vdim, _stream())


# -- what stands around the plain recurrence for gated linear attention and state-space layers (csrc/linear_recurrence.cu)

def gla_prep(proj, q_off: int, k_off: int, v_off: int, heads: int, dim: int, vdim: int, q_scale: float, tau: float, z_bias,
             qn, kn, vn, decay) -> None:
    """q (times q_scale), k and v columns of `proj` as float32 rows qn, kn [T, heads * dim], vn [T, heads * vdim];
    `decay` float32 [T, >= heads * dim] comes in as the raw decay projection z and leaves as
    sigmoid(z + z_bias)^(1 / tau) per head and key channel."""
    _dev(proj, z_bias, qn, kn, vn, decay)
    T = proj.shape[0]
    nqk, nv = heads * dim, heads * vdim
    _need(proj.dim() == 2 and proj.stride(1) == 1 and max(q_off + nqk, k_off + nqk, v_off + nv) <= proj.shape[1],
          "gla_prep: columns outside the projection")
    for t, n in ((qn, nqk), (kn, nqk), (vn, nv)):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.shape == (T, n), "gla_prep: outputs must be float32 [T, n]")
    _need(decay.dtype == torch.float32 and decay.dim() == 2 and decay.stride(1) == 1 and decay.shape[0] == T and
          decay.shape[1] >= nqk, "gla_prep: decay must be float32 [T, >= heads * dim]")
    _need(z_bias is None or (z_bias.dtype == torch.float32 and z_bias.numel() == nqk), "gla_prep: the bias must be float32 [heads * dim]")
    call("tie_gla_prep", dtype_code(proj), proj.data_ptr(), proj.stride(0), q_off, k_off, v_off, T, heads, dim, vdim,
         float(q_scale), float(tau), _ptr(z_bias), qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), decay.data_ptr(),
         decay.stride(0), _stream())


def ssd_prep(proj, c_off: int, b_off: int, x_off: int, dt_off: int, conv_w, conv_b, state, conv_state_off: int, seq_of_row,
             query_start, state_slots, heads: int, groups: int, state_size: int, vdim: int, taps: int, dt_bias, a_log,
             cn, bn, xn, dt, decay) -> None:
    """Short causal convolution (+ bias) and SiLU of the C, B and x columns of `proj` (conv_w float32 [channels, taps],
    channels in the order C, B, x; the last tap weighs the current token) to float32 cn, bn [T, groups * state_size] and
    xn [T, heads * vdim]; dt = softplus(proj[dt_off + h] + dt_bias[h]) and decay = exp(-exp(a_log[h]) dt), float32 [T, heads].
    `state` [slots, floats] holds, from conv_state_off on, each sequence's last taps - 1 convolution inputs."""
    _dev(proj, conv_w, conv_b, state, seq_of_row, query_start, state_slots, dt_bias, a_log, cn, bn, xn, dt, decay)
    T = proj.shape[0]
    ngn, nv = groups * state_size, heads * vdim
    _need(proj.dim() == 2 and proj.stride(1) == 1 and max(c_off + ngn, b_off + ngn, x_off + nv, dt_off + heads) <= proj.shape[1],
          "ssd_prep: columns outside the projection")
    _need(conv_w.dtype == torch.float32 and conv_w.is_contiguous() and conv_w.shape == (2 * ngn + nv, taps),
          "ssd_prep: convolution weights must be float32 [channels, taps]")
    _need(conv_b is None or (conv_b.dtype == torch.float32 and conv_b.numel() == 2 * ngn + nv), "ssd_prep: convolution bias must be float32 [channels]")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1 and
          conv_state_off + (taps - 1) * (2 * ngn + nv) <= state.shape[1], "ssd_prep: state rows too short")
    for t, n in ((cn, ngn), (bn, ngn), (xn, nv), (dt, heads), (decay, heads)):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.shape == (T, n), "ssd_prep: outputs must be float32 [T, n]")
    for t in (seq_of_row, query_start, state_slots):
        _need(t.dtype == torch.int32, "ssd_prep: index tensors must be int32")
    for t in (dt_bias, a_log):
        _need(t.dtype == torch.float32 and t.numel() == heads, "ssd_prep: dt_bias and a_log must be float32 [heads]")
    call("tie_ssd_prep", dtype_code(proj), proj.data_ptr(), proj.stride(0), c_off, b_off, x_off, dt_off, conv_w.data_ptr(),
         _ptr(conv_b), state.data_ptr(), state.stride(0), conv_state_off, seq_of_row.data_ptr(), query_start.data_ptr(),
         state_slots.data_ptr(), T, heads, groups, state_size, vdim, taps, dt_bias.data_ptr(), a_log.data_ptr(),
         cn.data_ptr(), bn.data_ptr(), xn.data_ptr(), dt.data_ptr(), decay.data_ptr(), _stream())


GATE_SIGMOID, GATE_SILU = 0, 1


def head_norm_gate(o, gate, weight, eps: float, out, heads: int, vdim: int, act: int = GATE_SIGMOID) -> None:
    """out[t, h] = (o[t, h] / rms(o[t, h])) * weight * act(gate[t, h]) per head of vdim; o float32, gate (rows may be
    strided) and out in the compute dtype; act GATE_SIGMOID or GATE_SILU."""
    _dev(o, gate, weight, out)
    T = o.shape[0]
    _need(o.dtype == torch.float32 and o.is_contiguous() and o.shape == (T, heads * vdim), "head_norm_gate: o must be float32 [T, heads * vdim]")
    _need(gate.dim() == 2 and gate.stride(1) == 1 and gate.shape == o.shape and gate.dtype == out.dtype,
          "head_norm_gate: gate must be [T, heads * vdim] in out's dtype")
    _need(weight.dtype == torch.float32 and weight.numel() == vdim, "head_norm_gate: weight must be float32 [vdim]")
    _need(out.is_contiguous() and out.shape == o.shape, "head_norm_gate: out must be [T, heads * vdim] contiguous")
    call("tie_head_norm_gate", dtype_code(out), o.data_ptr(), gate.data_ptr(), gate.stride(0), weight.data_ptr(), float(eps),
         out.data_ptr(), T, heads, vdim, int(act), _stream())


def ssd_out(o, xn, z, skip, weight, eps: float, out, heads: int, vdim: int, parts: int) -> None:
    """out = norm_parts((o + skip[h] xn) * silu(z)) * weight: the gate comes before the norm, and each of `parts` equal
    parts of the row is divided by its own root mean square. o, xn float32 [T, heads * vdim]; z (rows may be strided)
    and out in the compute dtype; skip float32 [heads]; weight float32 [heads * vdim]."""
    _dev(o, xn, z, skip, weight, out)
    T, inner = o.shape[0], heads * vdim
    for t in (o, xn):
        _need(t.dtype == torch.float32 and t.is_contiguous() and t.shape == (T, inner), "ssd_out: o and xn must be float32 [T, heads * vdim]")
    _need(z.dim() == 2 and z.stride(1) == 1 and z.shape == (T, inner) and z.dtype == out.dtype, "ssd_out: z must be [T, heads * vdim] in out's dtype")
    _need(skip.dtype == torch.float32 and skip.numel() == heads and weight.dtype == torch.float32 and weight.numel() == inner,
          "ssd_out: skip float32 [heads], weight float32 [heads * vdim]")
    _need(out.is_contiguous() and out.shape == (T, inner), "ssd_out: out must be [T, heads * vdim] contiguous")
    call("tie_ssd_out", dtype_code(out), o.data_ptr(), xn.data_ptr(), z.data_ptr(), z.stride(0), skip.data_ptr(),
         weight.data_ptr(), float(eps), out.data_ptr(), T, heads, vdim, int(parts), _stream())


# -- attention over one latent per token (csrc/attention_latent.cu) and products batched over heads

def latent_prep(proj, q_off: int, q_rank: int, kv_off: int, rank: int, rot: int, wq, wkv, eps: float, inv_freq, positions,
                slots, cq, k_cache) -> None:
    """From the stacked down-projections of every token: cq [T, q_rank] = rmsnorm(proj[q_off:]) * wq; the key plane's row
    at the token's slot = [rmsnorm(proj[kv_off : kv_off + rank]) * wkv | rotation of the `rot` columns behind them]."""
    _dev(proj, wq, wkv, inv_freq, positions, slots, cq, k_cache)
    T = proj.shape[0]
    _need(proj.dim() == 2 and proj.stride(1) == 1 and max(q_off + q_rank, kv_off + rank + rot) <= proj.shape[1],
          "latent_prep: columns outside the projection")
    _need(wq.dtype == torch.float32 and wq.numel() == q_rank and wkv.dtype == torch.float32 and wkv.numel() == rank,
          "latent_prep: norm weights must be float32 of the latents' sizes")
    _need(rot == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and 2 * inv_freq.numel() == rot),
          "latent_prep: inv_freq must be float32 [rot / 2]")
    _need(positions.dtype == torch.int32 and positions.numel() == T and slots.dtype == torch.int32 and slots.numel() == T,
          "latent_prep: positions and slots must be int32 [T]")
    _need(cq.shape == (T, q_rank) and cq.is_contiguous() and cq.dtype == proj.dtype, "latent_prep: cq must be [T, q_rank] contiguous")
    _need(k_cache.dim() == 4 and k_cache.is_contiguous() and k_cache.shape[1] == 1 and k_cache.shape[3] == rank + rot and
          k_cache.dtype == proj.dtype, "latent_prep: the key plane must be [pages, 1, page_size, rank + rot]")
    call("tie_latent_prep", dtype_code(proj), proj.data_ptr(), proj.stride(0), q_off, q_rank, kv_off, rank, rot, wq.data_ptr(),
         wkv.data_ptr(), float(eps), _ptr(inv_freq), positions.data_ptr(), slots.data_ptr(), cq.data_ptr(), k_cache.data_ptr(),
         T, _stream())


def latent_query_rot(q, dim: int, rot: int, inv_freq, positions, folded, rank: int, heads: int) -> None:
    """folded[t, h, rank : rank + rot] = rotation of q[t, h, dim : dim + rot] (heads of dim + rot in q, of rank + rot in folded)."""
    _dev(q, inv_freq, positions, folded)
    T = q.shape[0]
    _need(q.dim() == 2 and q.stride(1) == 1 and q.shape[1] >= heads * (dim + rot) and folded.dim() == 2 and folded.stride(1) == 1
          and folded.shape == (T, heads * (rank + rot)) and folded.dtype == q.dtype, "latent_query_rot: q [T, heads * (dim + rot)], folded [T, heads * (rank + rot)]")
    _need(rot == 0 or (inv_freq is not None and inv_freq.dtype == torch.float32 and 2 * inv_freq.numel() == rot),
          "latent_query_rot: inv_freq must be float32 [rot / 2]")
    _need(positions.dtype == torch.int32 and positions.numel() == T, "latent_query_rot: positions must be int32 [T]")
    call("tie_latent_query_rot", dtype_code(q), q.data_ptr(), q.stride(0), dim, rot, _ptr(inv_freq), positions.data_ptr(),
         folded.data_ptr(), folded.stride(0), rank, heads, T, _stream())


def attention_latent_mma_takes(q, k_cache, key_dim: int, rank: int) -> bool:
    """Whether the tensor-core kernels for attention over one cached row per token take these operands."""
    return (q.dtype == torch.bfloat16 and k_cache.dtype == torch.bfloat16 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0
            and bool(library.library().tie_attention_latent_mma_takes(key_dim, rank)))


def _latent_common(q, k_cache, query_start, context_lens, block_tables, heads, key_dim, rank):
    _need(k_cache.dim() == 4 and k_cache.is_contiguous() and k_cache.shape[1] == 1 and k_cache.shape[3] == key_dim and
          k_cache.dtype == torch.bfloat16, "latent attention: the key plane must be bfloat16 [pages, 1, page_size, key_dim]")
    _need(q.dim() == 2 and q.stride(1) == 1 and q.shape[1] >= heads * key_dim and q.dtype == torch.bfloat16,
          "latent attention: q must be bfloat16 [T, heads * key_dim]")
    S = context_lens.numel()
    _need(query_start.dtype == torch.int32 and query_start.numel() == S + 1 and context_lens.dtype == torch.int32 and
          block_tables.dtype == torch.int32 and block_tables.dim() == 2 and block_tables.shape[0] == S and block_tables.is_contiguous(),
          "latent attention: index tensors must be int32 (query_start [S+1], context_lens [S], block_tables [S, max_blocks])")


def attention_latent_prompt(q, k_cache, out, query_start, context_lens, block_tables, n_seqs: int, max_queries: int, heads: int,
                            key_dim: int, rank: int, scale: float, window: int = 0) -> None:
    """Attention of the first n_seqs sequences of the step (each brings several tokens; their rows come first) over a
    keys-only cache: every head reads the same rows of key_dim, a key's first `rank` elements are its value.
    q [T, heads * key_dim], out [T, heads * rank], bfloat16, on the tensor cores; softmax in float."""
    _dev(q, k_cache, out, query_start, context_lens, block_tables)
    _latent_common(q, k_cache, query_start, context_lens, block_tables, heads, key_dim, rank)
    _need(out.shape == (q.shape[0], heads * rank) and out.is_contiguous() and out.dtype == torch.bfloat16,
          "latent attention: out must be bfloat16 [T, heads * rank] contiguous")
    call("tie_attention_latent_prompt", q.data_ptr(), q.stride(0), k_cache.data_ptr(), out.data_ptr(), query_start.data_ptr(),
         context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], n_seqs, max_queries, heads, key_dim, rank,
         k_cache.shape[2], int(window), float(scale), _stream())


def attention_latent_split(q, k_cache, out, query_start, context_lens, block_tables, heads: int, key_dim: int, rank: int,
                           scale: float, seq_list, n_list: int, split_keys: int, max_splits: int, scratch, window: int = 0) -> None:
    """The same for sequences that bring one token each, their keys cut into splits of `split_keys` that are merged in
    split order; scratch holds attention_split_scratch_floats(n_list, heads, rank, max_splits) floats."""
    _dev(q, k_cache, out, query_start, context_lens, block_tables, seq_list, scratch)
    _latent_common(q, k_cache, query_start, context_lens, block_tables, heads, key_dim, rank)
    _need(out.shape == (q.shape[0], heads * rank) and out.is_contiguous() and out.dtype == torch.bfloat16,
          "latent attention: out must be bfloat16 [T, heads * rank] contiguous")
    _need(seq_list.dtype == torch.int32 and seq_list.numel() >= n_list, "latent attention: seq_list must be int32 [n_list]")
    _need(scratch.dtype == torch.float32 and scratch.numel() >= attention_split_scratch_floats(n_list, heads, rank, max_splits),
          "latent attention: scratch too small")
    call("tie_attention_latent_split", q.data_ptr(), q.stride(0), k_cache.data_ptr(), query_start.data_ptr(),
         context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], heads, key_dim, rank, k_cache.shape[2],
         int(window), float(scale), seq_list.data_ptr(), n_list, split_keys, max_splits, scratch.data_ptr(), _stream())
    call("tie_attention_merge", dtype_code(out), out.data_ptr(), query_start.data_ptr(), context_lens.data_ptr(), heads, rank,
         int(window), seq_list.data_ptr(), n_list, split_keys, max_splits, scratch.data_ptr(), _stream())


def head_gate_mul(y, gate, heads: int, head_size: int) -> None:
    """y[t, h, :] *= sigmoid(gate[t, h]) in place: one gate per head. y [T, heads * head_size], gate [T, heads] (rows may be strided)."""
    _dev(y, gate)
    T = y.shape[0]
    _need(y.dim() == 2 and y.stride(1) == 1 and y.shape[1] == heads * head_size and gate.dim() == 2 and gate.stride(1) == 1 and
          gate.shape == (T, heads) and gate.dtype == y.dtype, "head_gate_mul: y [T, heads * head_size] and gate [T, heads] of one dtype")
    call("tie_head_gate_mul", dtype_code(y), y.data_ptr(), y.stride(0), gate.data_ptr(), gate.stride(0), T, heads, head_size, _stream())


HEADS_MMA_MIN_ROWS = 16     # up to this many tokens the CUDA-core kernel streams each head's weights once


def gemm_heads(a, w, out, heads: int) -> None:
    """out[t, h, :] = w[h] a[t, h, :] for every head: a [T, >= heads * K] with head h at column h * a_head (a_head =
    a.shape[1] // heads), w [heads, N, K] contiguous, out [T, heads * out_head] with the result in the first N
    columns of each head. Float accumulation; a and w of one dtype. bfloat16 with more than a few tokens and sizes in
    whole vectors runs on the tensor cores, everything else on the CUDA cores."""
    _dev(a, w, out)
    T = a.shape[0]
    _need(a.dim() == 2 and out.dim() == 2 and w.dim() == 3 and w.is_contiguous() and w.shape[0] == heads, "gemm_heads: a, out 2-D, w [heads, N, K]")
    _need(a.stride(1) == 1 and out.stride(1) == 1 and a.shape[1] % heads == 0 and out.shape[1] % heads == 0 and out.shape[0] == T,
          "gemm_heads: rows must hold whole heads")
    N, K = w.shape[1], w.shape[2]
    a_head, o_head = a.shape[1] // heads, out.shape[1] // heads
    _need(K <= a_head and N <= o_head and a.dtype == w.dtype, "gemm_heads: heads narrower than the product")
    if (T > HEADS_MMA_MIN_ROWS and a.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and
            library.library().tie_gemm_heads_mma_takes(a.data_ptr(), a.stride(0), a_head, w.data_ptr(), out.data_ptr(), out.stride(0),
                                                       o_head, N, K)):
        call("tie_gemm_heads_mma", a.data_ptr(), a.stride(0), a_head, w.data_ptr(), out.data_ptr(), out.stride(0), o_head, T, N, K,
             heads, _stream())
        return
    call("tie_gemm_simt_batched", dtype_code(a), dtype_code(out), a.data_ptr(), w.data_ptr(), out.data_ptr(), T, N, K,
         a.stride(0), K, out.stride(0), heads, a_head, N * K, o_head, _stream())


# -- the residual stream beside a second stream, gated units with biases (csrc/stream_glue.cu)

def add_concat(x, delta, other, out) -> None:
    """x += delta (float32, in place; delta a tensor in out's dtype, a SplitSum, or None), then out[t] = [x[t] | other[t]]."""
    part = None
    if isinstance(delta, SplitSum):
        part, delta = delta, None
        _need(part.M == x.shape[0] and part.N == x.shape[-1], "add_concat: partial sums do not match x")
    _dev(x, delta, other, out)
    T, D = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous() and other.dtype == torch.float32 and other.is_contiguous() and
          other.shape == x.shape, "add_concat: x and other must be float32 [T, D] contiguous")
    _need(out.shape == (T, 2 * D) and out.is_contiguous(), "add_concat: out must be [T, 2 D] contiguous")
    if delta is not None:
        _need(delta.dtype == out.dtype and delta.shape == x.shape and delta.is_contiguous(), "add_concat: delta must match x's shape and out's dtype")
    call("tie_add_concat", dtype_code(out), x.data_ptr(), _ptr(delta), part.partial.data_ptr() if part else 0,
         part.stride if part else 0, part.splits if part else 0, other.data_ptr(), out.data_ptr(), T, D, _stream())


ACT_SILU, ACT_GELU_TANH = 0, 1


def glu_biased(gate_up, bias_gate, bias_up, out, act: int = ACT_SILU) -> None:
    """out[t, i] = act(gate_up[t, i] + bias_gate[i]) * (gate_up[t, I + i] + bias_up[i]); out [T, >= I]: a wider out gets a
    1 in column I and zeros behind it (for a product whose weight carries its bias as column I)."""
    _dev(gate_up, bias_gate, bias_up, out)
    T, I = gate_up.shape[0], gate_up.shape[1] // 2
    _need(gate_up.dim() == 2 and gate_up.shape[1] == 2 * I and gate_up.is_contiguous() and out.is_contiguous() and out.shape[0] == T
          and out.shape[1] >= I and gate_up.dtype == out.dtype, "glu_biased: gate_up [T, 2I], out [T, >= I], one dtype, contiguous")
    for b in (bias_gate, bias_up):
        _need(b is None or (b.dtype == torch.float32 and b.numel() == I), "glu_biased: biases must be float32 [I]")
    call("tie_glu_biased", dtype_code(out), gate_up.data_ptr(), _ptr(bias_gate), _ptr(bias_up), out.data_ptr(), T, I, out.shape[1],
         int(act), _stream())


# -- experts (csrc/moe.cu)

ROUTE_SOFTMAX, ROUTE_SIGMOID = 0, 1


def moe_route(logits, top: int, groups: int, keep: int, ids, weights, score_fn: int = ROUTE_SOFTMAX, correction=None,
              group_top: int = 1, renorm: bool = True, weight_scale: float = 1.0) -> None:
    """Per token: scores over all experts (`score_fn`: a softmax over the experts, or a sigmoid each); choice scores = scores +
    `correction` (float32 [E], optional); the `keep` best of `groups` equal blocks of consecutive experts (a group counts as the
    sum of its `group_top` largest choice scores: 1 = its best member); the `top` best experts of those by choice score. ids
    int32 [T, top], weights float32 [T, top] = the chosen experts' scores, over their sum (+ 1e-20) with `renorm`, times `weight_scale`."""
    _dev(logits, ids, weights, correction)
    T, E = logits.shape
    _need(logits.dtype == torch.float32 and logits.stride(1) == 1, "moe_route: logits must be float32 rows")
    _need(ids.dtype == torch.int32 and ids.is_contiguous() and ids.shape == (T, top) and weights.dtype == torch.float32 and
          weights.is_contiguous() and weights.shape == (T, top), "moe_route: ids int32 [T, top], weights float32 [T, top]")
    _need(correction is None or (correction.dtype == torch.float32 and correction.numel() == E and correction.is_contiguous()),
          "moe_route: the correction must be float32 [experts]")
    call("tie_moe_route", logits.data_ptr(), logits.stride(0), T, E, top, groups, keep, int(score_fn), _ptr(correction),
         int(group_top), int(bool(renorm)), float(weight_scale), ids.data_ptr(), weights.data_ptr(), _stream())


def moe_max_tiles(pairs: int, experts: int, block_m: int) -> int:
    return int(library.library().tie_moe_max_tiles(pairs, experts, block_m))


def moe_align(ids, experts: int, block_m: int, sorted_pairs, tile_expert, meta) -> None:
    """Lists the (token, choice) pairs by expert, each expert's range a whole number of tiles of block_m rows (-1 pads);
    tile_expert[i] is tile i's expert, meta[0] the number of tiles. All int32, on the device."""
    _dev(ids, sorted_pairs, tile_expert, meta)
    pairs = ids.numel()
    tiles = moe_max_tiles(pairs, experts, block_m)
    _need(all(t.dtype == torch.int32 and t.is_contiguous() for t in (ids, sorted_pairs, tile_expert, meta)) and
          sorted_pairs.numel() >= tiles * block_m and tile_expert.numel() >= tiles and meta.numel() >= 1,
          "moe_align: int32 arrays, sorted_pairs and tile_expert long enough for the most tiles")
    call("tie_moe_align", ids.data_ptr(), pairs, experts, block_m, sorted_pairs.data_ptr(), tile_expert.data_ptr(), meta.data_ptr(), _stream())


def moe_gemm(a, w, out, top: int, block_m: int, sorted_pairs, tile_expert, meta, max_tiles: int, second: bool = False,
             partial=None, weights=None, blocks_of=None) -> None:
    """Grouped products by expert. w [experts, N, K]. First (second False): a [T, K], out [T * top, N] = w[expert] a[token]
    per pair. Second: a [T * top, K], partial float32 [top, T, N] gets weights[pair] * (w[expert] a[pair]). With
    `blocks_of` = (N, K) and block_m 4, w is the experts' rows one after the other in k-blocks (`pack_k_blocks`)."""
    _dev(a, w, out, partial, weights, sorted_pairs, tile_expert, meta)
    w_rows = 0
    if blocks_of is not None:
        N, K = blocks_of
        _need(block_m == 4 and w.dim() == 3 and w.is_contiguous() and w.shape[2] == 64 and w.shape[0] == (K + 63) // 64 and
              w.shape[1] % N == 0 and a.dim() == 2 and a.stride(1) == 1 and a.shape[1] == K and a.dtype == w.dtype,
              "moe_gemm: weights in k-blocks of [experts * N, K] go with tiles of 4 rows")
        w_rows = w.shape[1]
    else:
        _need(w.dim() == 3 and w.is_contiguous() and a.dim() == 2 and a.stride(1) == 1 and a.shape[1] == w.shape[2] and a.dtype == w.dtype,
              "moe_gemm: w [experts, N, K] contiguous, a [rows, K] of w's dtype")
        N, K = w.shape[1], w.shape[2]
    if second:
        T = a.shape[0] // top
        _need(partial is not None and partial.dtype == torch.float32 and partial.is_contiguous() and partial.numel() >= top * T * N
              and weights is not None and weights.dtype == torch.float32 and weights.numel() == T * top,
              "moe_gemm: the second product needs partial float32 [top, T, N] and weights float32 [T * top]")
    else:
        T = a.shape[0]
        _need(out is not None and out.dim() == 2 and out.stride(1) == 1 and out.shape == (T * top, N) and out.dtype == a.dtype,
              "moe_gemm: out must be [T * top, N] in a's dtype")
    call("tie_moe_gemm", dtype_code(a), 1 if second else 0, block_m, a.data_ptr(), a.stride(0), w.data_ptr(), N * K,
         _ptr(out), out.stride(0) if out is not None else 0, _ptr(partial), T * N if second else 0, _ptr(weights),
         sorted_pairs.data_ptr(), tile_expert.data_ptr(), meta.data_ptr(), max_tiles, top, N, K, w_rows, _stream())


GROUPED_TILE = 128      # rows of a tile of the grouped product on the tensor cores


def moe_gather(h, sorted_pairs, meta, top: int, out) -> None:
    """out[r] = h[pair(r) // top] for the rows r listed by `moe_align` with tiles of GROUPED_TILE (zeros where a row pads a
    tile); bfloat16, width in whole 16-byte vectors."""
    _dev(h, sorted_pairs, meta, out)
    _need(h.dim() == 2 and h.stride(1) == 1 and out.dim() == 2 and out.is_contiguous() and out.shape[1] == h.shape[1] and
          h.dtype == torch.bfloat16 and out.dtype == torch.bfloat16, "moe_gather: bfloat16 rows of one width")
    call("tie_moe_gather", dtype_code(h), h.data_ptr(), h.stride(0), sorted_pairs.data_ptr(), meta.data_ptr(), GROUPED_TILE, top,
         out.data_ptr(), h.shape[1], out.shape[0], _stream())


def moe_combine(y, sorted_pairs, meta, top: int, weights, partial, tokens: int) -> None:
    """partial[pair % top][pair // top] = weights[pair] * y[row of the pair] (float32 [top, tokens, width])."""
    _dev(y, sorted_pairs, meta, weights, partial)
    _need(y.dim() == 2 and y.is_contiguous() and y.dtype == torch.bfloat16 and partial.dtype == torch.float32 and
          partial.numel() >= top * tokens * y.shape[1] and weights.dtype == torch.float32, "moe_combine: y bfloat16 rows, partial float32 [top, tokens, width]")
    call("tie_moe_combine", dtype_code(y), y.data_ptr(), sorted_pairs.data_ptr(), meta.data_ptr(), GROUPED_TILE, top,
         weights.data_ptr(), partial.data_ptr(), tokens * y.shape[1], y.shape[1], y.shape[0], _stream())


def gemm_grouped_takes(rows: int, N: int, K: int) -> bool:
    """Whether the grouped product on the tensor cores takes these sizes (bfloat16, k in whole 16-byte vectors)."""
    return K % 8 == 0 and N % 8 == 0 and rows % GROUPED_TILE == 0


def gemm_grouped(a, w_blocks, out, N: int, K: int, meta, tile_group) -> None:
    """out[r, :N] = w[group of r's tile] a[r] for the first meta[0] tiles of GROUPED_TILE rows of a; `w_blocks` is the
    groups' weights one after the other, [groups * N, K], stored in k-blocks (`pack_k_blocks`)."""
    _dev(a, w_blocks, out, meta, tile_group)
    _need(a.dim() == 2 and a.stride(1) == 1 and a.shape[1] == K and a.dtype == torch.bfloat16 and a.shape[0] % GROUPED_TILE == 0,
          "gemm_grouped: a must be bfloat16 [whole tiles, K]")
    _need(w_blocks.dim() == 3 and w_blocks.is_contiguous() and w_blocks.shape[2] == 64 and w_blocks.shape[0] == (K + 63) // 64 and
          w_blocks.shape[1] % N == 0 and w_blocks.dtype == torch.bfloat16, "gemm_grouped: weights must be k-blocks of [groups * N, K]")
    _need(out.dim() == 2 and out.stride(1) == 1 and out.shape == (a.shape[0], N), "gemm_grouped: out must be [rows, N]")
    bn = 256 if N >= 256 else 128
    call("tie_gemm_tc_grouped", dtype_code(out), a.data_ptr(), w_blocks.data_ptr(), out.data_ptr(), a.shape[0], N, K, a.stride(0),
         out.stride(0), bn, w_blocks.shape[1], meta.data_ptr(), tile_group.data_ptr(), _stream())


# -- layers whose sublayers read the stream side by side, and what stands around them (csrc/parallel_layer.cu)

def _delta_args(delta, x, what: str):
    """(tensor pointer, partial sums pointer, stride, splits) of a sublayer's output: a tensor, a SplitSum or None."""
    if delta is None:
        return 0, 0, 0, 0
    if isinstance(delta, SplitSum):
        _need(delta.M == x.shape[0] and delta.N == x.shape[1], f"{what}: partial sums do not match x")
        return 0, delta.partial.data_ptr(), delta.stride, delta.splits
    _need(delta.shape == x.shape and delta.is_contiguous(), f"{what}: a delta must have x's shape")
    return delta.data_ptr(), 0, 0, 0


def pair_hash_add(x, table, tokens, positions, seq_of_row, query_start, state_slots, prev_state, buckets: int, mul_prev: int,
                  mul_cur: int) -> None:
    """x[t] += table[(prev * mul_prev + token * mul_cur) mod buckets], prev the token before t in its sequence; a sequence's
    first token takes row `buckets`. `prev_state` int32 [slots] carries a request's last token from step to step."""
    _dev(x, table, tokens, positions, seq_of_row, query_start, state_slots, prev_state)
    T, D = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous(), "pair_hash_add: x must be float32 contiguous")
    _need(table.dim() == 2 and table.shape == (buckets + 1, D) and table.is_contiguous(), "pair_hash_add: the table must be [buckets + 1, D]")
    _need(prev_state.dtype == torch.int32 and prev_state.is_contiguous(), "pair_hash_add: the state must be int32")
    for t in (tokens, positions, seq_of_row, query_start, state_slots):
        _need(t.dtype == torch.int32, "pair_hash_add: index arrays must be int32")
    call("tie_pair_hash_add", dtype_code(table), x.data_ptr(), table.data_ptr(), tokens.data_ptr(), positions.data_ptr(),
         seq_of_row.data_ptr(), query_start.data_ptr(), state_slots.data_ptr(), prev_state.data_ptr(), int(buckets), int(mul_prev),
         int(mul_cur), T, D, _stream())


def add_row_vector(x, vec) -> None:
    """x[t] += vec for every row; both float32."""
    _dev(x, vec)
    _need(x.dtype == torch.float32 and x.is_contiguous() and vec.dtype == torch.float32 and vec.is_contiguous() and
          vec.numel() == x.shape[1], "add_row_vector: x float32 [T, D], vec float32 [D]")
    call("tie_add_row_vector", x.data_ptr(), vec.data_ptr(), x.shape[0], x.shape[1], _stream())


def group_norm_taps(x, groups: int, eps: float, w_a, out_a, w_b=None, out_b=None, taps_a=None, taps_b=None, ctx=None, unit=None,
                    ring=None, delta=None, rows=None, tile: int = 0) -> None:
    """u = x / rms over each of `groups` equal parts of a row; out_a = w_a * (u_t + sum_j taps_a[j] u_(t - taps + 1 + j)) (taps_a
    float32 [taps, D]: tap j of every channel side by side) and
    likewise out_b (optional): a grouped RMS norm whose output passes h + conv(h), a causal convolution over time per channel.
    With taps, `ctx` gives the step's index arrays, `ring` [slots, taps - 1, D] float32 the unit rows of earlier steps (by
    position mod taps - 1) and `unit` [T, D] receives the rows that `parallel_finish` moves into the ring. Without taps it is the
    grouped norm alone: `delta` (tensor or SplitSum) is added to x first and `rows` gathers (x is then left as it is). `tile`:
    rows a block with taps (0: chosen by the number of rows; the result does not depend on it)."""
    T, D = x.shape
    taps = 0 if taps_a is None else taps_a.shape[0]
    _dev(x, w_a, w_b, out_a, out_b, taps_a, taps_b, unit, ring, rows)
    _need(x.dtype == torch.float32 and x.is_contiguous(), "group_norm_taps: x must be float32 contiguous")
    n = out_a.shape[0]
    _need(out_a.shape[1] == D and out_a.is_contiguous() and (out_b is None or (out_b.shape == out_a.shape and out_b.is_contiguous()
                                                                              and out_b.dtype == out_a.dtype)),
          "group_norm_taps: outputs must be [n, D] contiguous of one dtype")
    for w in (w_a, w_b):
        _need(w is None or (w.dtype == torch.float32 and w.numel() == D), "group_norm_taps: norm weights must be float32 [D]")
    _need((w_b is None) == (out_b is None), "group_norm_taps: the second output needs a weight and a buffer")
    for tw in (taps_a, taps_b):
        _need(tw is None or (tw.dtype == torch.float32 and tw.shape == (taps, D) and tw.is_contiguous()),
              "group_norm_taps: taps must be float32 [taps, D]")
    if rows is None:
        _need(n == T, "group_norm_taps: out must have x's rows")
    else:
        _need(rows.dtype == torch.int32 and rows.numel() == n, "group_norm_taps: rows must be int32 [n]")
    dp, pp, ps, sp = _delta_args(delta, x, "group_norm_taps")
    if delta is not None and not isinstance(delta, SplitSum):
        _need(delta.dtype == out_a.dtype, "group_norm_taps: delta must have out's dtype")
    if taps > 1:
        _need(unit is not None and unit.dtype == torch.float32 and unit.shape == (T, D) and unit.is_contiguous() and
              ring is not None and ring.dtype == torch.float32 and ring.dim() == 3 and ring.shape[1:] == (taps - 1, D) and
              ring.is_contiguous(), "group_norm_taps: unit float32 [T, D], ring float32 [slots, taps - 1, D]")
    idx = (ctx.seq_of_row, ctx.positions, ctx.query_start, ctx.context_lens, ctx.state_slots) if taps > 0 else (None,) * 5
    call("tie_group_norm_taps", dtype_code(out_a), x.data_ptr(), dp, pp, ps, sp, _ptr(rows), n, D, int(groups), float(eps),
         w_a.data_ptr(), _ptr(w_b), _ptr(taps_a), _ptr(taps_b), taps, out_a.data_ptr(), _ptr(out_b), _ptr(unit), _ptr(ring),
         *(_ptr(t) for t in idx), int(tile), _stream())


def parallel_finish(x, mult: float, delta_a, delta_b, dtype, ctx=None, side=None, eps: float = 0.0, unit=None, ring=None) -> None:
    """x += mult * (delta_a + delta_b) (each a tensor of `dtype`, a SplitSum or None), in float32. With `side` = (table
    [vocab, n], gate [n, D], proj [D, n], norm float32 [D]) in `dtype`: g = gelu_tanh(gate x) * table[token], y = proj g,
    x += mult * y / rms(y) * norm. With `ring`: the rows of `unit` that are a sequence's last ring.shape[1] positions after
    this step go into the request's ring (what `group_norm_taps` left there)."""
    T, D = x.shape
    _dev(x, unit, ring)
    _need(x.dtype == torch.float32 and x.is_contiguous(), "parallel_finish: x must be float32 contiguous")
    for d in (delta_a, delta_b):
        _need(d is None or isinstance(d, SplitSum) or d.dtype == dtype, "parallel_finish: a delta tensor must be of the compute dtype")
    a, b = _delta_args(delta_a, x, "parallel_finish"), _delta_args(delta_b, x, "parallel_finish")
    n = 0
    table = gate = proj = norm = None
    if side is not None:
        table, gate, proj, norm = side
        _dev(table, gate, proj, norm)
        n = gate.shape[0]
        _need(table.dim() == 2 and table.shape[1] == n and gate.shape == (n, D) and proj.shape == (D, n) and
              all(t.is_contiguous() and t.dtype == dtype for t in (table, gate, proj)) and norm.dtype == torch.float32 and
              norm.numel() == D, "parallel_finish: side input tensors do not fit")
    R = 0 if ring is None else ring.shape[1]
    if R:
        _need(ring.dtype == torch.float32 and ring.is_contiguous() and ring.shape[2] == D and unit is not None and
              unit.dtype == torch.float32 and unit.shape == (T, D) and unit.is_contiguous(), "parallel_finish: ring float32 [slots, R, D], unit float32 [T, D]")
    need_ctx = R > 0 or side is not None
    call("tie_parallel_finish", F32 if dtype == torch.float32 else BF16, x.data_ptr(), T, D, float(mult), *a, *b,
         ctx.tokens.data_ptr() if need_ctx else 0, _ptr(table), _ptr(gate), _ptr(proj), _ptr(norm), n, float(eps), _ptr(unit) if R else 0,
         _ptr(ring) if R else 0, R, *((ctx.seq_of_row.data_ptr(), ctx.positions.data_ptr(), ctx.context_lens.data_ptr(),
                                      ctx.state_slots.data_ptr()) if need_ctx else (0, 0, 0, 0)), _stream())


def parallel_sum(x, mult: float, delta_a, delta_b, copy) -> None:
    """x += mult * (delta_a + delta_b) in float32 (each a tensor of copy's dtype, a SplitSum or None); copy = x in its own dtype."""
    _dev(x, copy)
    _need(x.dtype == torch.float32 and x.is_contiguous() and copy.shape == x.shape and copy.is_contiguous(),
          "parallel_sum: x float32 contiguous, copy of the same shape")
    for d in (delta_a, delta_b):
        _need(d is None or isinstance(d, SplitSum) or d.dtype == copy.dtype, "parallel_sum: a delta tensor must be of the compute dtype")
    a, b = _delta_args(delta_a, x, "parallel_sum"), _delta_args(delta_b, x, "parallel_sum")
    call("tie_parallel_sum", dtype_code(copy), x.data_ptr(), copy.data_ptr(), x.shape[0], x.shape[1], float(mult), *a, *b, _stream())


def side_gate_act(pre, table, tokens, g) -> None:
    """g[t] = gelu_tanh(pre[t]) * table[tokens[t]]: pre float32 [T, n], table [vocab, n] and g [T, n] of one dtype."""
    _dev(pre, table, tokens, g)
    T, n = pre.shape
    _need(pre.dtype == torch.float32 and pre.is_contiguous() and g.shape == (T, n) and g.is_contiguous() and table.dim() == 2 and
          table.shape[1] == n and table.is_contiguous() and table.dtype == g.dtype and tokens.dtype == torch.int32 and
          tokens.numel() >= T, "side_gate_act: pre float32 [T, n], table [vocab, n], g [T, n], tokens int32 [T]")
    call("tie_side_gate_act", dtype_code(g), pre.data_ptr(), table.data_ptr(), tokens.data_ptr(), g.data_ptr(), T, n, _stream())


def side_finish(x, y, mult: float, eps: float, norm, ctx=None, unit=None, ring=None) -> None:
    """x += mult * y / rms(y) * norm, all float32; with `ring`, the ring update of `parallel_finish`."""
    _dev(x, y, norm, unit, ring)
    T, D = x.shape
    _need(x.dtype == torch.float32 and x.is_contiguous() and y.dtype == torch.float32 and y.shape == x.shape and y.is_contiguous() and
          norm.dtype == torch.float32 and norm.numel() == D, "side_finish: x, y float32 [T, D], norm float32 [D]")
    R = 0 if ring is None else ring.shape[1]
    if R:
        _need(ring.dtype == torch.float32 and ring.is_contiguous() and ring.shape[2] == D and unit is not None and
              unit.dtype == torch.float32 and unit.shape == (T, D) and unit.is_contiguous(), "side_finish: ring float32 [slots, R, D], unit float32 [T, D]")
    call("tie_side_finish", x.data_ptr(), y.data_ptr(), T, D, float(mult), float(eps), norm.data_ptr(), _ptr(unit) if R else 0,
         _ptr(ring) if R else 0, R, *((ctx.seq_of_row.data_ptr(), ctx.positions.data_ptr(), ctx.context_lens.data_ptr(),
                                      ctx.state_slots.data_ptr()) if R else (0, 0, 0, 0)), _stream())


# -- attention whose scores are mixed across heads, with a sink (csrc/attention_mixed.cu)

def rope_pairs_unit_append(proj, q_off: int, k_off: int, v_off: int, inv_freq, unit: bool, eps: float, positions, slots, k_cache,
                           v_cache, q_heads: int, kv_heads: int, dim: int, vdim: int) -> None:
    """proj [T, ...] holds q, k and v of every token at columns q_off, k_off, v_off. The first 2 * len(inv_freq) dimensions of each
    q and k head are turned in neighbouring pairs (2i, 2i+1) by position * inv_freq[i]; with `unit` each head is then divided by
    its root mean square; q goes back in place, k and v into the cache planes at the token's slot."""
    _dev(proj, inv_freq, positions, slots, k_cache, v_cache)
    T = proj.shape[0]
    _need(proj.dim() == 2 and proj.stride(1) == 1 and q_off + q_heads * dim <= proj.shape[1] and k_off + kv_heads * dim <= proj.shape[1]
          and v_off + kv_heads * vdim <= proj.shape[1], "rope_pairs_unit_append: q, k or v outside the projection")
    _need(positions.dtype == torch.int32 and positions.numel() == T and slots.dtype == torch.int32 and slots.numel() == T,
          "rope_pairs_unit_append: positions and slots must be int32 [T]")
    _need(inv_freq is None or (inv_freq.dtype == torch.float32 and inv_freq.is_contiguous()), "rope_pairs_unit_append: inv_freq must be float32")
    _check_kv_planes(k_cache, v_cache, kv_heads, dim, vdim)
    _need(k_cache.dtype == proj.dtype, "rope_pairs_unit_append: dtype differs from the cache's")
    call("tie_rope_pairs_unit_append", dtype_code(proj), proj.data_ptr(), proj.stride(0), q_off, k_off, v_off, _ptr(inv_freq),
         2 * inv_freq.numel() if inv_freq is not None else 0, int(bool(unit)), float(eps), positions.data_ptr(), slots.data_ptr(),
         k_cache.data_ptr(), v_cache.data_ptr(), T, q_heads, kv_heads, dim, vdim, k_cache.shape[2], _stream())


def attention_mixed(q, k_cache, v_cache, out, mix, ctx_arrays, rows: int, heads: int, kv_heads: int, dim: int, vdim: int, scale: float,
                    sink: bool, seq_list=None, n_list: int = 0, split_keys: int = 0, max_splits: int = 0, scratch=None) -> None:
    """Causal attention over the paged cache with scores mixed across heads (`mix` float32 [heads, heads] or None) and, with
    `sink`, one more key of score 0 without a value in every softmax. `ctx_arrays` = (seq_of_row, query_start, context_lens,
    block_tables). Rows [0, rows) each against the keys up to their own position; or, with `seq_list`, one row per listed
    sequence with its keys in splits of `split_keys` that are merged in split order (scratch:
    attention_split_scratch_floats(n_list, heads, vdim, max_splits) floats)."""
    seq_of_row, query_start, context_lens, block_tables = ctx_arrays
    _dev(q, k_cache, v_cache, out, mix, seq_of_row, query_start, context_lens, block_tables, seq_list, scratch)
    _attn_common_dv(q, k_cache, v_cache, out, query_start, context_lens, block_tables, heads, kv_heads, dim, vdim)
    _need(mix is None or (mix.dtype == torch.float32 and mix.shape == (heads, heads) and mix.is_contiguous()),
          "attention_mixed: mix must be float32 [heads, heads]")
    split = seq_list is not None
    if split:
        _need(seq_list.dtype == torch.int32 and seq_list.numel() >= n_list, "attention_mixed: seq_list must be int32 [n_list]")
        _need(scratch is not None and scratch.dtype == torch.float32 and
              scratch.numel() >= attention_split_scratch_floats(n_list, heads, vdim, max_splits), "attention_mixed: scratch too small")
    else:
        _need(seq_of_row.dtype == torch.int32 and seq_of_row.numel() >= rows and rows <= q.shape[0], "attention_mixed: seq_of_row must be int32 [T]")
    call("tie_attention_mixed", dtype_code(q), q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
         _ptr(mix), seq_of_row.data_ptr(), query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(),
         block_tables.shape[1], rows, heads, kv_heads, dim, vdim, k_cache.shape[2], float(scale), int(bool(sink)),
         _ptr(seq_list) if split else 0, n_list, split_keys, max_splits, _ptr(scratch) if split else 0, _stream())
    if split and n_list > 0:
        call("tie_attention_merge", dtype_code(out), out.data_ptr(), query_start.data_ptr(), context_lens.data_ptr(), heads, vdim,
             0, seq_list.data_ptr(), n_list, split_keys, max_splits, scratch.data_ptr(), _stream())


def attention_mixed_tc_takes(heads: int, kv_heads: int, dim: int, vdim: int) -> bool:
    """Whether `attention_mixed_tc` serves this geometry (bfloat16 only); the CUDA-core kernel serves every geometry."""
    return bool(library.library().tie_attention_mixed_tc_takes(int(heads), int(kv_heads), int(dim), int(vdim)))


def attention_mixed_tc(q, k_cache, v_cache, out, mix, query_start, context_lens, block_tables, n_seqs: int, max_queries: int,
                       heads: int, kv_heads: int, dim: int, vdim: int, scale: float, sink: bool, seq_list=None, split_keys: int = 0,
                       max_splits: int = 0, scratch=None) -> None:
    """`attention_mixed` in bfloat16 on the tensor cores: for the rows of sequences 0 .. n_seqs-1, each bringing several tokens
    (at most `max_queries`); or, with `seq_list` (int32 [n_seqs]), one row per listed sequence with its keys in splits of
    `split_keys` (a multiple of 64) that are merged in split order (scratch as for `attention_mixed`)."""
    _dev(q, k_cache, v_cache, out, mix, query_start, context_lens, block_tables, seq_list, scratch)
    _attn_common_dv(q, k_cache, v_cache, out, query_start, context_lens, block_tables, heads, kv_heads, dim, vdim)
    _need(q.dtype == torch.bfloat16, "attention_mixed_tc: bfloat16 only")
    _need(mix is None or (mix.dtype == torch.float32 and mix.shape == (heads, heads) and mix.is_contiguous()),
          "attention_mixed_tc: mix must be float32 [heads, heads]")
    split = seq_list is not None
    if split:
        _need(seq_list.dtype == torch.int32 and seq_list.numel() >= n_seqs, "attention_mixed_tc: seq_list must be int32 [n_seqs]")
        _need(scratch is not None and scratch.dtype == torch.float32 and
              scratch.numel() >= attention_split_scratch_floats(n_seqs, heads, vdim, max_splits), "attention_mixed_tc: scratch too small")
    call("tie_attention_mixed_tc", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), _ptr(mix),
         query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], int(n_seqs),
         int(max_queries), heads, kv_heads, dim, vdim, k_cache.shape[2], float(scale), int(bool(sink)),
         _ptr(seq_list) if split else 0, int(split_keys), int(max_splits), _ptr(scratch) if split else 0, _stream())
    if split and n_seqs > 0:
        call("tie_attention_merge", dtype_code(out), out.data_ptr(), query_start.data_ptr(), context_lens.data_ptr(), heads, vdim,
             0, seq_list.data_ptr(), n_seqs, split_keys, max_splits, scratch.data_ptr(), _stream())


# -- a norm without statistics and a sinusoid on the embedding (csrc/tanh_norm.cu)

class ScaledSum:
    """Sublayer outputs that join the residual stream together, each with a factor: sum_i scale_i * term_i, a term a
    tensor [T, D] in the compute dtype or a SplitSum. Norms that say `takes_scaled_sum` add the terms in float32 while
    they read them; `materialize` adds them into a tensor for everyone else."""

    def __init__(self, terms):
        self.terms = [(t, float(c)) for t, c in terms if t is not None]
        if not 1 <= len(self.terms) <= 2:
            raise InvalidArgument(f"a scaled sum has one or two terms, got {len(self.terms)}")

    def materialize(self, out: torch.Tensor) -> torch.Tensor:
        acc = torch.zeros(out.shape, dtype=torch.float32, device=out.device)      # off the product path: toy parts and tests only
        for t, c in self.terms:
            if isinstance(t, SplitSum):
                t = t.partial[:t.splits * t.stride].view(t.splits, t.M, t.N).sum(dim=0)
            acc += c * t.float()
        out.copy_(acc)
        return out


def add_tanh_norm(x: torch.Tensor, delta, alpha: float, weight: torch.Tensor, bias: torch.Tensor, out: torch.Tensor, rows=None) -> None:
    """x += delta (when given; float32, in place), out = tanh(alpha x) * weight + bias in out's dtype. `delta`: a tensor in
    out's dtype, a SplitSum, or a ScaledSum of up to two of those. With `rows` (int32 [R]) out[i] comes from row rows[i]
    and x is left as it is."""
    terms = delta.terms if isinstance(delta, ScaledSum) else ([(delta, 1.0)] if delta is not None else [])
    _dev(x, weight, bias, out, rows)
    D, n = x.shape[-1], out.shape[0]
    _need(x.dtype == torch.float32 and x.is_contiguous(), "add_tanh_norm: x must be float32 contiguous")
    _need(all(w.dtype == torch.float32 and w.numel() == D for w in (weight, bias)), "add_tanh_norm: weight and bias must be float32 [D]")
    _need(out.shape[-1] == D and out.is_contiguous(), "add_tanh_norm: out must be [n, D] contiguous")
    _need(rows is None and n == x.shape[0] or rows is not None and rows.dtype == torch.int32 and rows.numel() == n,
          "add_tanh_norm: out must have x's rows, or rows must be int32 [n]")
    args = []
    for t, c in terms + [(None, 0.0)] * (2 - len(terms)):
        if isinstance(t, SplitSum):
            _need(t.M == x.shape[0] and t.N == D, "add_tanh_norm: partial sums do not match x")
            args += [0, t.partial.data_ptr(), t.stride, t.splits, c]
        else:
            if t is not None:
                _dev(t)
                _need(t.dtype == out.dtype and t.shape == x.shape and t.is_contiguous(), "add_tanh_norm: a delta must match x's shape and out's dtype")
            args += [_ptr(t), 0, 0, 0, c]
    call("tie_add_tanh_norm", dtype_code(out), x.data_ptr(), *args, _ptr(rows), float(alpha), weight.data_ptr(), bias.data_ptr(),
         out.data_ptr(), n, D, _stream())


def sinusoid_add(x: torch.Tensor, positions: torch.Tensor, base: float = 10000.0) -> None:
    """x[t, 2i] += sin(p * base^(-2i/D)), x[t, 2i+1] += cos of the same angle, p = positions[t]; x float32 [T, D]."""
    _dev(x, positions)
    _need(x.dtype == torch.float32 and x.is_contiguous() and x.dim() == 2, "sinusoid_add: x must be float32 [T, D] contiguous")
    _need(positions.dtype == torch.int32 and positions.numel() >= x.shape[0], "sinusoid_add: positions must be int32 [T]")
    call("tie_sinusoid_add", x.data_ptr(), positions.data_ptr(), x.shape[0], x.shape[1], float(base), _stream())


def two_branch_unit(z: torch.Tensor, out: torch.Tensor, c_pos: float, c_neg: float) -> None:
    """out = c_pos z^2 + z/2 where z > 0, else c_neg (exp(z) - 1 - z) + z/2; z and out alike, contiguous."""
    _dev(z, out)
    _need(z.shape == out.shape and z.dtype == out.dtype and z.is_contiguous() and out.is_contiguous(), "two_branch_unit: z and out alike, contiguous")
    call("tie_two_branch_unit", dtype_code(z), z.data_ptr(), out.data_ptr(), z.numel(), float(c_pos), float(c_neg), _stream())


# -- attention whose query heads read slices of wider key rows (csrc/attention_simt.cu, csrc/score_maps.cu)

def slice_norm_append(proj, q_off: int, nq: int, k_off: int, nk: int, v_off: int, v_width: int, dim: int, wq, wk, eps: float,
                      slots, k_cache, v_cache) -> None:
    """Per token of `proj` [T, width]: the nq slices of `dim` from column q_off are divided by their root mean square and
    multiplied by wq (float32 [dim]; None: left alone), in place; with planes given, the nk slices from k_off likewise with
    wk on their way into the key plane [pages, heads, page, k_row] and the v_width columns from v_off into the value plane
    [pages, heads, page, v_row] at slots[t] (negative: nothing is written)."""
    _dev(proj, wq, wk, slots, k_cache, v_cache)
    T = proj.shape[0]
    _need(proj.dim() == 2 and proj.stride(1) == 1, "slice_norm_append: proj rows must be contiguous")
    for w in (wq, wk):
        _need(w is None or (w.dtype == torch.float32 and w.numel() == dim), "slice_norm_append: a norm weight must be float32 [dim]")
    write = k_cache is not None
    heads = k_row = v_row = page = 0
    if write:
        _need(k_cache.dim() == 4 and v_cache.dim() == 4 and k_cache.is_contiguous() and v_cache.is_contiguous() and
              k_cache.shape[:3] == v_cache.shape[:3] and k_cache.dtype == proj.dtype and v_cache.dtype == proj.dtype,
              "slice_norm_append: planes [pages, heads, page, size] in proj's dtype")
        heads, page, k_row, v_row = k_cache.shape[1], k_cache.shape[2], k_cache.shape[3], v_cache.shape[3]
        _need(slots.dtype == torch.int32 and slots.numel() >= T, "slice_norm_append: slots must be int32 [T]")
    call("tie_slice_norm_append", dtype_code(proj), proj.data_ptr(), proj.stride(0), q_off, nq, k_off, nk, v_off, v_width, dim, _ptr(wq),
         _ptr(wk), float(eps), _ptr(slots), _ptr(k_cache), _ptr(v_cache), T, heads, k_row, v_row, page, 1 if write else 0, _stream())


def _maps_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, dim, sub_count):
    _need(k_cache.dim() == 4 and v_cache.dim() == 4 and k_cache.is_contiguous() and v_cache.is_contiguous() and
          k_cache.shape[:3] == v_cache.shape[:3] and k_cache.dtype == q.dtype and v_cache.dtype == q.dtype,
          "attention maps: planes [pages, heads, page, size] in q's dtype")
    kv_heads, v_dim = k_cache.shape[1], v_cache.shape[3]
    _need(k_cache.shape[3] >= sub_count * dim, "attention maps: key rows too short for their slices")
    _need(q.dim() == 2 and q.stride(1) == 1 and q.shape[1] >= q_heads * dim, "attention maps: q too narrow")
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (q.shape[0], q_heads * v_dim),
          "attention maps: out must be float32 [T, q_heads * value row]")
    S = context_lens.numel()
    _need(query_start.dtype == torch.int32 and query_start.numel() == S + 1 and context_lens.dtype == torch.int32 and
          block_tables.dtype == torch.int32 and block_tables.dim() == 2 and block_tables.shape[0] == S and block_tables.is_contiguous(),
          "attention maps: query_start int32 [S+1], context_lens int32 [S], block_tables int32 [S, blocks]")
    return S, kv_heads, v_dim


def attention_maps_rows(q, k_cache, v_cache, out, seq_of_row, query_start, context_lens, block_tables, rows: int, q_heads: int, dim: int,
                        group: int, sub_div: int, sub_count: int, scale: float, window: int = 0, chunk: int = 0, softcap: float = 0.0, r1=None,
                        r2=None) -> None:
    """The first `rows` rows of q, each over all keys it sees. Query head h reads cached head (h // group) % cached heads and, of
    that key row, the `dim` elements from ((h // sub_div) % sub_count) * dim; its softmax weights meet the whole value row.
    `chunk` > 0: a position sees its own chunk of that many positions only; `softcap` > 0: score <- cap tanh(score / cap);
    r1, r2 (float32 [q_heads]): score -= r1 ln(1 + r2 distance). out float32 [T, q_heads * value row]."""
    _dev(q, k_cache, v_cache, out, seq_of_row, query_start, context_lens, block_tables, r1, r2)
    S, kv_heads, v_dim = _maps_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, dim, sub_count)
    call("tie_attention_maps_rows", dtype_code(q), q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
         seq_of_row.data_ptr(), query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1],
         int(rows), S, q_heads, kv_heads, dim, k_cache.shape[3], int(sub_div), int(sub_count), v_dim, k_cache.shape[2], int(window),
         int(chunk), float(scale), float(softcap), _ptr(r1), _ptr(r2), int(group), _stream())


def attention_maps_split(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads: int, dim: int, group: int, sub_div: int,
                         sub_count: int, scale: float, seq_list, n_list: int, split_keys: int, max_splits: int, scratch, window: int = 0,
                         chunk: int = 0, softcap: float = 0.0, r1=None, r2=None) -> None:
    """The same for the sequences of seq_list, which bring one row each, their keys cut into splits of split_keys; scratch holds
    attention_split_scratch_floats(n_list, q_heads, value row, max_splits) floats."""
    _dev(q, k_cache, v_cache, out, query_start, context_lens, block_tables, seq_list, scratch, r1, r2)
    S, kv_heads, v_dim = _maps_common(q, k_cache, v_cache, out, query_start, context_lens, block_tables, q_heads, dim, sub_count)
    _need(scratch.dtype == torch.float32 and scratch.numel() >= attention_split_scratch_floats(n_list, q_heads, v_dim, max_splits),
          "attention maps: scratch too small")
    call("tie_attention_maps_split", dtype_code(q), q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(),
         query_start.data_ptr(), context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], S, q_heads, kv_heads, dim,
         k_cache.shape[3], int(sub_div), int(sub_count), v_dim, k_cache.shape[2], int(window), int(chunk), float(scale), float(softcap),
         _ptr(r1), _ptr(r2), int(group), seq_list.data_ptr(), n_list, split_keys, max_splits, scratch.data_ptr(), _stream())


def attention_prompt_maps_takes(q, k_cache, v_cache, dim: int) -> bool:
    """Whether prompt portions of this geometry run on the tensor cores: bfloat16, slices of 64, 128 or 256 for keys and values
    alike, pages that are powers of two from 8 up, rows in whole 16-byte pieces."""
    page = k_cache.shape[2]
    return (q.dtype == torch.bfloat16 and dim in (64, 128, 256) and page >= 8 and page & (page - 1) == 0 and k_cache.shape[3] % dim == 0 and
            v_cache.shape[3] % dim == 0 and q.stride(0) % 8 == 0 and q.data_ptr() % 16 == 0 and os.environ.get("TIE_NO_MAPS_TC") != "1")


def attention_prompt_maps(q, k_cache, v_cache, out, query_start, context_lens, block_tables, n_seqs: int, max_queries: int, q_heads: int,
                          kv_heads: int, dim: int, scale: float, v_shift: int = 0, chunk: int = 0, softcap: float = 0.0, r1=None, r2=None) -> None:
    """Prompt portions on the tensor cores (TMA-fed `mma.sync`, float scores and softmax, weights as two bfloat16 terms) for score
    maps over slices of wider cached rows: kv head v of `kv_heads` reads cached head v % cached heads, its `dim` key elements from column
    (v // cached heads) * dim and its `dim` value elements from column ((v // cached heads + v_shift) % slices) * dim, slices = value row / dim;
    query heads v * (q_heads / kv_heads) .. read kv head v. out float32 [T, q_heads, slices, dim]: the call fills the slice of its value
    column. At most 16 query heads a kv head."""
    _dev(q, k_cache, v_cache, out, query_start, context_lens, block_tables, r1, r2)
    slices = v_cache.shape[3] // dim
    _need(out.dtype == torch.float32 and out.is_contiguous() and out.shape == (q.shape[0], q_heads * slices * dim),
          "attention_prompt_maps: out must be float32 [T, q_heads * slices * dim]")
    _need(q_heads % kv_heads == 0 and q_heads // kv_heads <= 16 and kv_heads % k_cache.shape[1] == 0, "attention_prompt_maps: impossible head counts")
    call("tie_attention_prompt_maps", q.data_ptr(), q.stride(0), k_cache.data_ptr(), v_cache.data_ptr(), out.data_ptr(), query_start.data_ptr(),
         context_lens.data_ptr(), block_tables.data_ptr(), block_tables.shape[1], n_seqs, max_queries, q_heads, kv_heads, dim, k_cache.shape[2],
         k_cache.shape[0], 0, float(scale), k_cache.shape[1], k_cache.shape[3], v_cache.shape[3], int(v_shift), int(chunk), float(softcap),
         _ptr(r1), _ptr(r2), _stream())


def diff_combine(a, gate, lam: float, mult: float, eps: float, out, heads: int, vdim: int) -> None:
    """a [T, 2 * heads * vdim] (map 1 of every head, then map 2; float32 or the compute dtype): o = a1 - lam a2;
    out = (o / rms(o)) * mult * sigmoid(gate) per head; gate (None: no gate; rows may be strided) and out [T, heads * vdim] in the compute dtype."""
    _dev(a, gate, out)
    T = a.shape[0]
    _need(a.dtype in (torch.float32, out.dtype) and a.is_contiguous() and a.shape == (T, heads * 2 * vdim), "diff_combine: a must be [T, 2 * heads * vdim], float32 or out's dtype")
    _need(out.is_contiguous() and out.shape == (T, heads * vdim), "diff_combine: out must be [T, heads * vdim] contiguous")
    _need(gate is None or (gate.dim() == 2 and gate.stride(1) == 1 and gate.shape == out.shape and gate.dtype == out.dtype),
          "diff_combine: gate must be [T, heads * vdim] in out's dtype")
    call("tie_diff_combine", dtype_code(out), int(a.dtype == torch.float32), a.data_ptr(), _ptr(gate), gate.stride(0) if gate is not None else 0, float(lam), float(mult),
         float(eps), out.data_ptr(), T, heads, vdim, _stream())


def head_talk(a, talk, out, heads: int, kv_heads: int, vdim: int) -> None:
    """a [T, heads * kv_heads * vdim] (float32 or the compute dtype; every head's weights on every kv head's values): out[t, h] = sum_g talk[h, g] *
    a[t, g, kv head of h]; talk float32 [heads, heads]; out [T, heads * vdim] in the compute dtype."""
    _dev(a, talk, out)
    T = a.shape[0]
    _need(a.dtype in (torch.float32, out.dtype) and a.is_contiguous() and a.shape == (T, heads * kv_heads * vdim), "head_talk: a must be [T, heads * kv_heads * vdim], float32 or out's dtype")
    _need(talk.dtype == torch.float32 and talk.is_contiguous() and talk.shape == (heads, heads), "head_talk: talk must be float32 [heads, heads]")
    _need(out.is_contiguous() and out.shape == (T, heads * vdim), "head_talk: out must be [T, heads * vdim] contiguous")
    call("tie_head_talk", dtype_code(out), int(a.dtype == torch.float32), a.data_ptr(), talk.data_ptr(), out.data_ptr(), T, heads, kv_heads, vdim, _stream())


# -- a recurrence that blends its inputs with the token before (csrc/time_mix.cu, csrc/delta_rule.cu)

def token_shift_concat(h, state, prev_off: int, ctx, out) -> None:
    """out[t] = [h[t] | h[t - 1]]; the row before a portion's first row comes from the sequence's row of `state` (float32
    [slots, floats], at prev_off; zeros at position 0). h [T, D] and out [T, 2 D] in the compute dtype, contiguous."""
    _dev(h, state, out)
    T, D = h.shape
    _need(h.is_contiguous() and out.dtype == h.dtype and out.is_contiguous() and out.shape == (T, 2 * D), "token_shift_concat: out must be [T, 2 D] in h's dtype")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1 and state.shape[1] >= prev_off + D, "token_shift_concat: state rows too short")
    call("tie_token_shift_concat", dtype_code(h), h.data_ptr(), state.data_ptr(), state.stride(0), prev_off, ctx.seq_of_row.data_ptr(),
         ctx.query_start.data_ptr(), ctx.positions.data_ptr(), ctx.state_slots.data_ptr(), out.data_ptr(), T, D, _stream())


def time_mix_prep(proj, r_off: int, k_off: int, v_off: int, inner_off: int, w2t, w0, rn, kn, vn, decay) -> None:
    """Columns r_off.., k_off.., v_off.. of `proj` (n each) as float32 rows rn, kn, vn; decay = exp(-exp(tanh(inner) w2t + w0)) with
    `inner` the columns inner_off.. of proj (as many as w2t has rows), w2t float32 [inner, n], w0 float32 [n]."""
    _dev(proj, w2t, w0, rn, kn, vn, decay)
    T, n = decay.shape
    rank = w2t.shape[0]
    _need(proj.dim() == 2 and proj.stride(1) == 1 and proj.shape[0] == T and proj.shape[1] >= max(r_off, k_off, v_off) + n and
          proj.shape[1] >= inner_off + rank, "time_mix_prep: proj too narrow")
    _need(all(t.dtype == torch.float32 and t.is_contiguous() and t.shape == (T, n) for t in (rn, kn, vn, decay)) and w0.dtype == torch.float32 and
          w0.numel() == n and w2t.dtype == torch.float32 and w2t.is_contiguous() and w2t.shape == (rank, n),
          "time_mix_prep: float32 [T, n] outputs, w2t float32 [inner, n], w0 float32 [n]")
    call("tie_time_mix_prep", dtype_code(proj), proj.data_ptr(), proj.stride(0), r_off, k_off, v_off, inner_off, rank, w2t.data_ptr(), w0.data_ptr(),
         rn.data_ptr(), kn.data_ptr(), vn.data_ptr(), decay.data_ptr(), T, n, _stream())


def delta_rule_bonus(qn, kn, vn, decay, bonus, state, ctx, heads: int, dim: int, out) -> None:
    """The plain recurrence read before it is written: per head o_t = (S + diag(bonus) k_t v_t^T)^T q_t, then
    S <- diag(decay_t) S + k_t v_t^T. qn, kn, vn, decay, out float32 [T, heads * dim]; bonus float32 [heads * dim]; S [heads, dim, dim]
    sits at the start of the sequence's row of `state`."""
    _dev(qn, kn, vn, decay, bonus, state, out)
    T = qn.shape[0]
    _need(all(t.dtype == torch.float32 and t.is_contiguous() and t.shape == (T, heads * dim) for t in (qn, kn, vn, decay, out)),
          "delta_rule_bonus: float32 [T, heads * dim] rows")
    _need(bonus.dtype == torch.float32 and bonus.is_contiguous() and bonus.numel() == heads * dim, "delta_rule_bonus: bonus must be float32 [heads * dim]")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1 and state.shape[1] >= heads * dim * dim,
          "delta_rule_bonus: state rows too short")
    call("tie_delta_rule_bonus", F32, qn.data_ptr(), kn.data_ptr(), vn.data_ptr(), 0, decay.data_ptr(), decay.stride(0), state.data_ptr(),
         state.stride(0), heads * dim * dim, qn.data_ptr(), qn.stride(0), 0, 0, 0, ctx.query_start.data_ptr(), ctx.state_slots.data_ptr(),
         ctx.S, heads, heads, dim, dim, 1, out.data_ptr(), bonus.data_ptr(), _stream())


def time_mix_out(o, gate, weight, eps: float, out, heads: int, dim: int, h, state, prev_off: int, ctx) -> None:
    """out[t, hd] = (o[t, hd] / rms(o[t, hd])) * weight[hd] * silu(gate[t, hd]) per head of dim (weight float32 [heads * dim]); and the
    last row of h of every sequence becomes the row its slot keeps (state[slot, prev_off:prev_off + D], float32)."""
    _dev(o, gate, weight, out, h, state)
    T, D = h.shape
    _need(o.dtype == torch.float32 and o.is_contiguous() and o.shape == (T, heads * dim), "time_mix_out: o must be float32 [T, heads * dim]")
    _need(gate.dim() == 2 and gate.stride(1) == 1 and gate.shape == o.shape and gate.dtype == out.dtype and out.is_contiguous() and
          out.shape == o.shape, "time_mix_out: gate and out [T, heads * dim] in the compute dtype")
    _need(weight.dtype == torch.float32 and weight.numel() == heads * dim and h.is_contiguous() and h.dtype == out.dtype,
          "time_mix_out: weight float32 [heads * dim], h contiguous in the compute dtype")
    _need(state.dtype == torch.float32 and state.dim() == 2 and state.stride(1) == 1 and state.shape[1] >= prev_off + D, "time_mix_out: state rows too short")
    call("tie_time_mix_out", dtype_code(out), o.data_ptr(), gate.data_ptr(), gate.stride(0), weight.data_ptr(), float(eps), out.data_ptr(), T,
         heads, dim, h.data_ptr(), D, state.data_ptr(), state.stride(0), prev_off, ctx.seq_of_row.data_ptr(), ctx.query_start.data_ptr(),
         ctx.state_slots.data_ptr(), _stream())
