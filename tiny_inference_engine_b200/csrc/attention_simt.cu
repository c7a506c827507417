// Causal attention over the paged cache on the CUDA cores, for any head size that is a
// multiple of 8, any number of heads and groups, any page size; float or bfloat16 storage,
// float scores, softmax and accumulation. It is the attention of the 32-bit path and the
// fallback of the bfloat16 path.
//
// What it computes is the reference's paged_attention (src/backend/cpu/cpu_backend.cpp:261-319):
// query row t of sequence s has position pos = context_len[s] - n_queries(s) + (t - query_start[s])
// and sees keys 0..pos (with a window w > 0: keys pos-w+1..pos); query head h reads kv head
// h / (Hq/Hkv); online softmax of scale * q.k; out = acc / l.
//
// Two kernels share the inner loop:
//   rows kernel   one warp per (row, head) over all of its keys: prompt portions.
//   split kernel  one warp per (sequence, head, split of the keys) for sequences that bring
//                 one token: each split of `split_keys` keys leaves (max, sum, acc) in
//                 scratch memory and a merge kernel combines them in split order. The split
//                 size is a constant of the call, so the order of the sums for a token
//                 depends only on its own context, never on the batch around it.
#include <math.h>

#include "common.cuh"
#include "launchers.h"

namespace tie {

struct AttnArgs {
  const void* q;            // [T, ...] row stride q_stride, head h at h * head_dim
  const void* k_cache;      // [pages, kv_heads, page_size, head_dim]
  const void* v_cache;
  void* out;                // [T, q_heads * head_dim]
  const int* seq_of_row;    // [T]
  const int* query_start;   // [S + 1]
  const int* context_lens;  // [S]
  const int* block_tables;  // [S, max_blocks]
  long long q_stride;
  int max_blocks;
  int rows;                 // T
  int seqs;                 // S
  int q_heads, kv_heads, head_dim, page_size;
  int window;               // 0 = all keys
  float scale;
  int v_dim;                // size of a value head (and of an output head); keys and queries have head_dim
  int v_ld;                 // elements between value rows; 0: v_dim. With the key plane given as the value plane too
                            // and v_ld = head_dim, a value is the first v_dim elements of its key (a latent cache).
  // Score maps over slices of wider key rows (all zero: the plain attention above). A key row holds k_ld elements, and
  // query head h reads the head_dim of them that start at ((h / sub_div) % sub_count) * head_dim: two score maps a head
  // over one value (sub_div 1, sub_count 2), or all kv heads' keys in one row so that every query head weights the
  // values of every kv head (sub_div = query heads per kv head, sub_count = kv heads, one cached head).
  int k_ld;                 // elements between key rows; 0: head_dim
  int sub_div, sub_count;
  int chunk;                // > 0: a position sees the keys of its own chunk of this many positions (counted from 0) only
  float softcap;            // > 0: score <- softcap * tanh(score / softcap)
  const float* r1;          // [q_heads] or null: score -= r1[h] * ln(1 + r2[h] * (position - key position))
  const float* r2;
  int out_f32;              // the output rows are float whatever the storage type
  int group;                // > 0: query head h reads cached head (h / group) % kv_heads (query heads laid out map by map)
};

// The first key that position `pos` sees.
__device__ __forceinline__ int first_visible(int pos, int window, int chunk) {
  if (chunk > 0) return pos / chunk * chunk;
  return window > 0 ? max(0, pos - window + 1) : 0;
}

// What a score passes on its way to the softmax beside the scale: a cap and a bias that grows with the distance.
struct ScoreShape {
  float softcap, r1, r2;
  int pos;                  // the query's position
};

// One warp: online softmax over keys [lo, hi] of one (query vector, kv head).
// q is in shared memory (float, already multiplied by nothing: scale is applied to the score).
// Lane `l` owns output dims [l * DPL, (l + 1) * DPL). Returns m, l and acc in registers.
template <typename T, int DPL>
__device__ __forceinline__ void attend_range(const float* __restrict__ qs, const T* __restrict__ kc,
                                             const T* __restrict__ vc, const int* __restrict__ table, int kvh,
                                             int kv_heads, int head_dim, int v_dim, int v_ld, int page_size, float scale,
                                             int lo, int hi, float& m, float& l, float (&acc)[DPL], int k_ld = 0, int k_off = 0,
                                             const ScoreShape shape = ScoreShape{0.0f, 0.0f, 0.0f, 0}) {
  if (k_ld == 0) k_ld = head_dim;
  // whole pieces of four value elements a lane, each on its own boundary
  const bool v_quads = DPL % 4 == 0 && v_dim % DPL == 0 && v_ld % 4 == 0 && reinterpret_cast<uintptr_t>(vc) % (4 * sizeof(T)) == 0;
  constexpr int V = Vec16<T>::N;
  const int lane = threadIdx.x & 31;
  const int d0 = lane * DPL;
  for (int base = lo; base <= hi; base += 32) {
    const int j = base + lane;
    const bool valid = j <= hi;
    int row = 0;  // index of the key's row: head_dim elements in the key plane, v_dim in the value plane
    float s = -INFINITY;
    if (valid) {
      const int page = table[j / page_size];
      row = (page * kv_heads + kvh) * page_size + j % page_size;
      const T* kr = kc + static_cast<long long>(row) * k_ld + k_off;
      float dot = 0.0f;
      if (head_dim % V == 0 && k_ld % V == 0) {      // rows of whole 16-byte pieces
        for (int d = 0; d < head_dim; d += V) {
          Vec16<T> kv;
          kv.load(kr + d);
#pragma unroll
          for (int e = 0; e < V; ++e) dot = fmaf(qs[d + e], kv.v[e], dot);
        }
      } else {
        for (int d = 0; d < head_dim; ++d) dot = fmaf(qs[d], ld(kr + d), dot);
      }
      s = scale * dot;
      if (shape.softcap > 0.0f) s = shape.softcap * tanhf(s / shape.softcap);
      if (shape.r1 != 0.0f) s -= shape.r1 * log1pf(shape.r2 * static_cast<float>(shape.pos - j));
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);  // m = -inf at the start gives 0
    const float p = valid ? expf(s - m_new) : 0.0f;
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int e = 0; e < DPL; ++e) acc[e] *= corr;
    const int count = min(32, hi - base + 1);
    if (DPL % 4 == 0 && v_quads) {
      // a lane's value elements in pieces of four, and the keys four at a time so that their loads are in flight together
      // (keys beyond `count` have weight 0 and row 0, which is real memory)
      const bool mine = d0 < v_dim;
#pragma unroll 4
      for (int jj = 0; jj < 32; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);       // every lane takes part in the exchanges
        const int rj = __shfl_sync(0xffffffffu, row, jj);
        if (mine) {
          const T* vr = vc + static_cast<long long>(rj) * v_ld + d0;
#pragma unroll
          for (int e4 = 0; e4 < DPL / 4; ++e4) {
            float v4[4];
            load4(vr + 4 * e4, v4);
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[4 * e4 + e] = fmaf(pj, v4[e], acc[4 * e4 + e]);
          }
        }
      }
    } else {
      for (int jj = 0; jj < count; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        const int rj = __shfl_sync(0xffffffffu, row, jj);
        if (d0 < v_dim) {
          const T* vr = vc + static_cast<long long>(rj) * v_ld + d0;
#pragma unroll
          for (int e = 0; e < DPL; ++e)
            if (d0 + e < v_dim) acc[e] = fmaf(pj, ld(vr + e), acc[e]);
        }
      }
    }
  }
}

__device__ __forceinline__ int kv_head_of(const AttnArgs& a, int h) {
  return a.group > 0 ? (h / a.group) % a.kv_heads : h / (a.q_heads / a.kv_heads);
}

__device__ __forceinline__ int key_offset(const AttnArgs& a, int h) {
  return a.sub_count > 1 ? ((h / a.sub_div) % a.sub_count) * a.head_dim : 0;
}

__device__ __forceinline__ ScoreShape score_shape(const AttnArgs& a, int h, int pos) {
  return ScoreShape{a.softcap, a.r1 ? a.r1[h] : 0.0f, a.r1 ? a.r2[h] : 0.0f, pos};
}

template <typename T, int DPL>
__global__ void __launch_bounds__(128) attention_rows_kernel(AttnArgs a) {
  pdl_sync();
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + warp;
  if (item >= static_cast<long long>(a.rows) * a.q_heads) return;
  const int t = static_cast<int>(item / a.q_heads);
  const int h = static_cast<int>(item % a.q_heads);
  const int s = a.seq_of_row[t];
  const int qs0 = a.query_start[s], qs1 = a.query_start[s + 1];
  const int pos = a.context_lens[s] - (qs1 - qs0) + (t - qs0);
  const int lo = first_visible(pos, a.window, a.chunk);
  const int kvh = kv_head_of(a, h);

  float* qs = smem + warp * a.head_dim;
  const T* qv = static_cast<const T*>(a.q) + static_cast<long long>(t) * a.q_stride + static_cast<long long>(h) * a.head_dim;
  for (int d = lane; d < a.head_dim; d += 32) qs[d] = ld(qv + d);
  __syncwarp();

  float m = -INFINITY, l = 0.0f, acc[DPL] = {};
  attend_range<T, DPL>(qs, static_cast<const T*>(a.k_cache), static_cast<const T*>(a.v_cache),
                       a.block_tables + static_cast<long long>(s) * a.max_blocks, kvh, a.kv_heads, a.head_dim,
                       a.v_dim, a.v_ld ? a.v_ld : a.v_dim, a.page_size, a.scale, lo, pos, m, l, acc, a.k_ld, key_offset(a, h),
                       score_shape(a, h, pos));
  const int d0 = lane * DPL;
  if (d0 < a.v_dim) {
    const long long at = (static_cast<long long>(t) * a.q_heads + h) * a.v_dim + d0;
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;  // no keys (a padding row): zeros
#pragma unroll
    for (int e = 0; e < DPL; ++e)
      if (d0 + e < a.v_dim) {
        if (a.out_f32) static_cast<float*>(a.out)[at + e] = acc[e] * inv;
        else st(static_cast<T*>(a.out) + at + e, acc[e] * inv);
      }
  }
}

// Split kernel: sequences listed in `seq_list` (each brings exactly one query row).
// scratch: [n_list, q_heads, max_splits, v_dim + 2] floats (acc, then m, l).
template <typename T, int DPL>
__global__ void __launch_bounds__(128) attention_split_kernel(AttnArgs a, const int* __restrict__ seq_list, int n_list,
                                                              int split_keys, int max_splits, float* __restrict__ scratch) {
  pdl_sync();
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.y;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + warp;
  if (item >= static_cast<long long>(n_list) * a.q_heads) return;
  const int li = static_cast<int>(item / a.q_heads);
  const int h = static_cast<int>(item % a.q_heads);
  const int s = seq_list[li];
  const int t = a.query_start[s];
  const int pos = a.context_lens[s] - 1;
  const int lo0 = first_visible(pos, a.window, a.chunk);
  const int lo = lo0 + split * split_keys;
  if (lo > pos) return;  // this sequence has fewer splits
  // The last split takes whatever is left, so that a context longer than max_splits * split_keys (a caller
  // who sized max_splits from something else than the longest context) costs time, never keys.
  const int hi = split == max_splits - 1 ? pos : min(pos, lo + split_keys - 1);
  const int kvh = kv_head_of(a, h);

  float* qs = smem + warp * a.head_dim;
  const T* qv = static_cast<const T*>(a.q) + static_cast<long long>(t) * a.q_stride + static_cast<long long>(h) * a.head_dim;
  for (int d = lane; d < a.head_dim; d += 32) qs[d] = ld(qv + d);
  __syncwarp();

  float m = -INFINITY, l = 0.0f, acc[DPL] = {};
  attend_range<T, DPL>(qs, static_cast<const T*>(a.k_cache), static_cast<const T*>(a.v_cache),
                       a.block_tables + static_cast<long long>(s) * a.max_blocks, kvh, a.kv_heads, a.head_dim,
                       a.v_dim, a.v_ld ? a.v_ld : a.v_dim, a.page_size, a.scale, lo, hi, m, l, acc, a.k_ld, key_offset(a, h),
                       score_shape(a, h, pos));
  float* dst = scratch + ((static_cast<long long>(li) * a.q_heads + h) * max_splits + split) * (a.v_dim + 2);
  const int d0 = lane * DPL;
  if (d0 < a.v_dim) {
#pragma unroll
    for (int e = 0; e < DPL; ++e)
      if (d0 + e < a.v_dim) dst[d0 + e] = acc[e];
  }
  if (lane == 0) {
    dst[a.v_dim] = m;
    dst[a.v_dim + 1] = l;
  }
}


// Single rows in splits, the heads of a cached head together: one block per (sequence, cached head, split), a warp per query head
// that reads that cached head. A tile of 32 keys (their whole key and value rows) comes into shared memory once and serves every
// warp: lane j scores key j against its head's slice of the key row, then the lanes share the value row's columns. Leaves
// (acc, max, sum) where attention_split_kernel leaves them, for the same merge.
constexpr int kGroupTile = 32;

// 16 bytes from global to shared memory without a stop in a register: all of a thread's copies of a tile are in flight together.
__device__ __forceinline__ void group_copy16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src) : "memory");
}

template <typename T, int DPL>
__global__ void __launch_bounds__(1024) attention_group_split_kernel(AttnArgs a, const int* __restrict__ seq_list, int n_list,
                                                                     int split_keys, int max_splits, float* __restrict__ scratch,
                                                                     int k_pad) {
  pdl_sync();
  extern __shared__ __align__(16) uint8_t group_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const int li = blockIdx.x / a.kv_heads, c = blockIdx.x % a.kv_heads, split = blockIdx.y;
  const int k_ld = a.k_ld ? a.k_ld : a.head_dim, v_ld = a.v_ld ? a.v_ld : a.v_dim;
  // shared memory: q of every warp (float), the tile's cache rows, K tile (rows padded by k_pad elements), V tile
  float* qs_all = reinterpret_cast<float*>(group_smem);
  int* rows = reinterpret_cast<int*>(qs_all + warps * a.head_dim);
  T* k_tile = reinterpret_cast<T*>(reinterpret_cast<uint8_t*>(rows + kGroupTile) + ((16 - (warps * a.head_dim + kGroupTile) * 4 % 16) % 16));
  const int k_row = k_ld + k_pad;
  T* v_tile = k_tile + kGroupTile * k_row;
  const int s = seq_list[li];
  const int t = a.query_start[s];
  const int pos = a.context_lens[s] - 1;
  const int lo0 = first_visible(pos, a.window, a.chunk);
  const int lo = lo0 + split * split_keys;
  if (lo > pos) return;                      // the whole block: this sequence has fewer splits
  const int hi = split == max_splits - 1 ? pos : min(pos, lo + split_keys - 1);
  // the warp's query head: the heads h with (h / group) % kv_heads == c, in order
  const int group = a.group > 0 ? a.group : a.q_heads / a.kv_heads;
  const int h = ((warp / group) * a.kv_heads + c) * group + warp % group;
  float* qs = qs_all + warp * a.head_dim;
  const T* qv = static_cast<const T*>(a.q) + static_cast<long long>(t) * a.q_stride + static_cast<long long>(h) * a.head_dim;
  for (int d = lane; d < a.head_dim; d += 32) qs[d] = ld(qv + d);
  const int k_off = key_offset(a, h);
  const ScoreShape shape = score_shape(a, h, pos);
  const int* table = a.block_tables + static_cast<long long>(s) * a.max_blocks;
  const T* kc = static_cast<const T*>(a.k_cache);
  const T* vc = static_cast<const T*>(a.v_cache);
  constexpr int V = Vec16<T>::N;
  const bool k_vec = k_ld % V == 0 && k_pad % V == 0 && reinterpret_cast<uintptr_t>(kc) % 16 == 0;
  const bool v_vec = v_ld % V == 0 && reinterpret_cast<uintptr_t>(vc) % 16 == 0;
  const bool dot_vec = k_vec && a.head_dim % V == 0;
  const int d0 = lane * DPL;
  float m = -INFINITY, l = 0.0f, acc[DPL] = {};
  for (int base = lo; base <= hi; base += kGroupTile) {
    __syncthreads();                          // everyone is through with the tile before
    if (threadIdx.x < kGroupTile) {
      const int j = base + threadIdx.x;
      rows[threadIdx.x] = j <= hi ? (table[j / a.page_size] * a.kv_heads + c) * a.page_size + j % a.page_size : -1;
    }
    __syncthreads();
    if (k_vec) {
      const int pieces = k_ld / V;
      for (int i = threadIdx.x; i < kGroupTile * pieces; i += blockDim.x) {
        const int kk = i / pieces, p = (i % pieces) * V;
        if (rows[kk] >= 0) group_copy16(k_tile + kk * k_row + p, kc + static_cast<long long>(rows[kk]) * k_ld + p);
        else *reinterpret_cast<uint4*>(k_tile + kk * k_row + p) = make_uint4(0u, 0u, 0u, 0u);
      }
    } else {
      for (int i = threadIdx.x; i < kGroupTile * k_ld; i += blockDim.x) {
        const int kk = i / k_ld, p = i % k_ld;
        k_tile[kk * k_row + p] = rows[kk] >= 0 ? kc[static_cast<long long>(rows[kk]) * k_ld + p] : T(0.0f);
      }
    }
    if (v_vec) {
      const int pieces = v_ld / V;
      for (int i = threadIdx.x; i < kGroupTile * pieces; i += blockDim.x) {
        const int kk = i / pieces, p = (i % pieces) * V;
        if (rows[kk] >= 0) group_copy16(v_tile + kk * v_ld + p, vc + static_cast<long long>(rows[kk]) * v_ld + p);
        else *reinterpret_cast<uint4*>(v_tile + kk * v_ld + p) = make_uint4(0u, 0u, 0u, 0u);
      }
    } else {
      for (int i = threadIdx.x; i < kGroupTile * v_ld; i += blockDim.x) {
        const int kk = i / v_ld, p = i % v_ld;
        v_tile[kk * v_ld + p] = rows[kk] >= 0 ? vc[static_cast<long long>(rows[kk]) * v_ld + p] : T(0.0f);
      }
    }
    asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");      // the copies of this thread; the barrier does the rest
    __syncthreads();
    const int j = base + lane;
    const bool valid = j <= hi;
    float sc = -INFINITY;
    if (valid) {
      const T* kr = k_tile + lane * k_row + k_off;
      float dot = 0.0f;
      if (dot_vec) {
        for (int d = 0; d < a.head_dim; d += V) {
          Vec16<T> kv;
          kv.load(kr + d);
#pragma unroll
          for (int e = 0; e < V; ++e) dot = fmaf(qs[d + e], kv.v[e], dot);
        }
      } else {
        for (int d = 0; d < a.head_dim; ++d) dot = fmaf(qs[d], ld(kr + d), dot);
      }
      sc = a.scale * dot;
      if (shape.softcap > 0.0f) sc = shape.softcap * tanhf(sc / shape.softcap);
      if (shape.r1 != 0.0f) sc -= shape.r1 * log1pf(shape.r2 * static_cast<float>(pos - j));
    }
    const float m_new = fmaxf(m, warp_max(sc));
    const float corr = expf(m - m_new);
    const float p = valid ? expf(sc - m_new) : 0.0f;
    l = l * corr + warp_sum(p);
    m = m_new;
#pragma unroll
    for (int e = 0; e < DPL; ++e) acc[e] *= corr;
    if (DPL % V == 0 && v_vec && a.v_dim % DPL == 0) {      // a lane's value elements in 16-byte pieces: no two lanes on a bank
      const bool mine = d0 < a.v_dim;
#pragma unroll 4
      for (int jj = 0; jj < kGroupTile; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        if (mine) {
          const T* vr = v_tile + jj * v_ld + d0;
#pragma unroll
          for (int ev = 0; ev < DPL / V; ++ev) {
            Vec16<T> vv;
            vv.load(vr + V * ev);
#pragma unroll
            for (int e = 0; e < V; ++e) acc[V * ev + e] = fmaf(pj, vv.v[e], acc[V * ev + e]);
          }
        }
      }
    } else if (DPL % 4 == 0 && v_ld % 4 == 0 && a.v_dim % DPL == 0) {      // in pieces of four
      const bool mine = d0 < a.v_dim;
#pragma unroll 4
      for (int jj = 0; jj < kGroupTile; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        if (mine) {
          const T* vr = v_tile + jj * v_ld + d0;
#pragma unroll
          for (int e4 = 0; e4 < DPL / 4; ++e4) {
            float v4[4];
            load4(vr + 4 * e4, v4);
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[4 * e4 + e] = fmaf(pj, v4[e], acc[4 * e4 + e]);
          }
        }
      }
    } else {
#pragma unroll 4
      for (int jj = 0; jj < kGroupTile; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, p, jj);
        const T* vr = v_tile + jj * v_ld + d0;
#pragma unroll
        for (int e = 0; e < DPL; ++e)
          if (d0 + e < a.v_dim) acc[e] = fmaf(pj, ld(vr + e), acc[e]);
      }
    }
  }
  float* dst = scratch + ((static_cast<long long>(li) * a.q_heads + h) * max_splits + split) * (a.v_dim + 2);
  if (d0 < a.v_dim) {
#pragma unroll
    for (int e = 0; e < DPL; ++e)
      if (d0 + e < a.v_dim) dst[d0 + e] = acc[e];
  }
  if (lane == 0) {
    dst[a.v_dim] = m;
    dst[a.v_dim + 1] = l;
  }
}

// The grouped kernel's launch geometry for `a`, or 0 bytes when it does not fit (then the kernel above serves).
template <typename T>
static size_t group_split_smem(const AttnArgs& a, int* warps, int* k_pad) {
  const int per = a.q_heads / a.kv_heads;
  const int k_ld = a.k_ld ? a.k_ld : a.head_dim, v_ld = a.v_ld ? a.v_ld : a.v_dim;
  *warps = per;
  *k_pad = 16 / static_cast<int>(sizeof(T));        // rows a 16-byte piece apart in the banks: lanes read a column of 16-byte pieces
  if (per > 32 || a.v_ld != 0 || a.v_dim > 1024) return 0;      // (64 registers a thread: no room for more than 32 sums a lane)
  const size_t bytes = static_cast<size_t>(per) * a.head_dim * 4 + kGroupTile * 4 + 16 +
                       static_cast<size_t>(kGroupTile) * (k_ld + *k_pad + v_ld) * sizeof(T);
  return bytes <= 96 * 1024 ? bytes : 0;
}

// Merge of the splits of one (sequence, head), in split order: one block each. The weights
// exp(m_i - m) of the splits are computed once into shared memory, then every thread sums its
// dims over the splits.
constexpr int kMergeThreads = 128;
constexpr int kMergeMaxSplits = 256;

template <typename T>
__global__ void __launch_bounds__(kMergeThreads) attention_merge_kernel(AttnArgs a, const int* __restrict__ seq_list,
                                                                        int n_list, int split_keys, int max_splits,
                                                                        const float* __restrict__ scratch) {
  pdl_sync();
  __shared__ float weight[kMergeMaxSplits];
  __shared__ float inv_l;
  const int item = blockIdx.x;
  const int li = item / a.q_heads, h = item % a.q_heads;
  const int s = seq_list[li];
  const int t = a.query_start[s];
  const int pos = a.context_lens[s] - 1;
  const long long at = (static_cast<long long>(t) * a.q_heads + h) * a.head_dim;
  T* o = static_cast<T*>(a.out) + at;
  float* of = static_cast<float*>(a.out) + at;
  if (pos < 0) {  // a padding sequence: no keys, zeros
    for (int d = threadIdx.x; d < a.head_dim; d += kMergeThreads) {
      if (a.out_f32) of[d] = 0.0f;
      else st(o + d, 0.0f);
    }
    return;
  }
  const int lo0 = first_visible(pos, a.window, a.chunk);
  const int splits = min((pos - lo0) / split_keys + 1, max_splits);   // the last one took the rest (split kernels)
  const int stride = a.head_dim + 2;
  const float* src = scratch + (static_cast<long long>(li) * a.q_heads + h) * max_splits * stride;
  if (threadIdx.x < 32) {
    float m = -INFINITY;
    for (int i = threadIdx.x; i < splits; i += 32) m = fmaxf(m, src[i * stride + a.head_dim]);
    m = warp_max(m);
    float l = 0.0f;
    for (int i = threadIdx.x; i < splits; i += 32) {
      const float w = expf(src[i * stride + a.head_dim] - m);
      weight[i] = w;
      l += src[i * stride + a.head_dim + 1] * w;   // summed below in a fixed lane order
    }
    l = warp_sum(l);
    if (threadIdx.x == 0) inv_l = l > 0.0f ? 1.0f / l : 0.0f;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < a.head_dim; d += kMergeThreads) {
    float acc = 0.0f;
    for (int i = 0; i < splits; ++i) acc = fmaf(src[i * stride + d], weight[i], acc);
    if (a.out_f32) of[d] = acc * inv_l;
    else st(o + d, acc * inv_l);
  }
}

template <typename T>
int launch_attention(const AttnArgs& a, const int* row_seq_unused, const int* seq_list, int n_list, int split_keys,
                     int max_splits, float* scratch, int rows_kernel, cudaStream_t s, bool grouped = false) {
  (void)row_seq_unused;
  int group_warps = 0, k_pad = 0;
  const size_t group_smem = grouped && !rows_kernel ? group_split_smem<T>(a, &group_warps, &k_pad) : 0;
  const int warps = 4;
  const size_t smem = static_cast<size_t>(warps) * a.head_dim * sizeof(float);
  AttnArgs merge_args = a;            // the merge kernel sees output heads only
  merge_args.head_dim = a.v_dim;
  const int dpl = (a.v_dim + 31) / 32;
#define TIE_ATTN_CASE(D)                                                                                         \
  do {                                                                                                           \
    if (rows_kernel) {                                                                                           \
      const long long items = static_cast<long long>(a.rows) * a.q_heads;                                        \
      if (items > 0) TIE_LAUNCH((attention_rows_kernel<T, D>), ceil_div(items, warps), warps * 32, smem, s, a);            \
    } else {                                                                                                     \
      const long long items = static_cast<long long>(n_list) * a.q_heads;                                        \
      if (items > 0) {                                                                                           \
        if (group_smem > 0) {                                                                                    \
          if (group_smem > 48 * 1024)                                                                            \
            cudaFuncSetAttribute(attention_group_split_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024); \
          TIE_LAUNCH((attention_group_split_kernel<T, D>), dim3(n_list * a.kv_heads, max_splits), group_warps * 32, group_smem, s, \
              a, seq_list, n_list, split_keys, max_splits, scratch, k_pad);                                      \
        } else                                                                                                   \
        TIE_LAUNCH((attention_split_kernel<T, D>), dim3(ceil_div(items, warps), max_splits), warps * 32, smem, s,           \
            a, seq_list, n_list, split_keys, max_splits, scratch);                                               \
        TIE_LAUNCH((attention_merge_kernel<T>), static_cast<int>(items), kMergeThreads, 0, s, merge_args, seq_list, n_list, split_keys, \
                                                                                    max_splits, scratch);         \
      }                                                                                                          \
    }                                                                                                            \
  } while (0)
  if (dpl <= 1) TIE_ATTN_CASE(1);
  else if (dpl <= 2) TIE_ATTN_CASE(2);
  else if (dpl <= 4) TIE_ATTN_CASE(4);
  else if (dpl <= 8) TIE_ATTN_CASE(8);
  else if (dpl <= 16) TIE_ATTN_CASE(16);
  else if (dpl <= 32) TIE_ATTN_CASE(32);
  else TIE_ATTN_CASE(64);
#undef TIE_ATTN_CASE
  TIE_RETURN_LAUNCH("paged_attention_simt");
}

}  // namespace tie

using namespace tie;

// `any_size`: the launchers for keys and values of two sizes take heads of any size (rows that are not whole
// 16-byte pieces are read element by element); the others keep the sizes that the tensor-core kernels share.
static int check_attn(const AttnArgs& a, bool any_size = false) {
  TIE_REQUIRE(a.q_heads > 0 && a.kv_heads > 0 && a.q_heads % a.kv_heads == 0,
              "attention: %d query heads are not a multiple of %d kv heads", a.q_heads, a.kv_heads);
  TIE_REQUIRE(a.head_dim > 0 && a.head_dim <= (any_size ? 1024 : 512), "attention: head_dim %d must be 1 to %d", a.head_dim,
              any_size ? 1024 : 512);
  if (!any_size) {
    TIE_REQUIRE(a.head_dim % 8 == 0, "attention: head_dim %d must be a multiple of 8 and at most 512", a.head_dim);
    TIE_REQUIRE(a.head_dim <= 256 || a.head_dim % 16 == 0, "attention: head_dim %d above 256 must be a multiple of 16",
                a.head_dim);
  }
  TIE_REQUIRE(a.v_dim > 0 && a.v_dim <= (any_size ? 2048 : 512), "attention: value heads of %d (1 to %d)", a.v_dim, any_size ? 2048 : 512);
  TIE_REQUIRE(a.page_size > 0 && a.max_blocks > 0, "attention: bad page geometry");
  TIE_REQUIRE(a.window >= 0, "attention: negative window");
  return kOk;
}

// All rows of the step, each over all of its keys (prompt portions and, when no split is
// wanted, single tokens too).
TIE_API int tie_attention_rows(int dtype, const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                               void* out, const int* seq_of_row, const int* query_start, const int* context_lens,
                               const int* block_tables, int max_blocks, int rows, int seqs, int q_heads, int kv_heads,
                               int head_dim, int page_size, int window, float scale, cudaStream_t s) {
  const AttnArgs a{q, k_cache, v_cache, out, seq_of_row, query_start, context_lens, block_tables, q_stride, max_blocks,
                   rows, seqs, q_heads, kv_heads, head_dim, page_size, window, scale, head_dim};
  if (const int st = check_attn(a)) return st;
  if (dtype == TIE_F32) return launch_attention<float>(a, nullptr, nullptr, 0, 0, 0, nullptr, 1, s);
  if (dtype == TIE_BF16) return launch_attention<__nv_bfloat16>(a, nullptr, nullptr, 0, 0, 0, nullptr, 1, s);
  set_error("attention: unknown dtype code %d", dtype);
  return kBadArgument;
}

// The sequences of seq_list bring one token each; their keys are cut into splits of
// `split_keys` keys. scratch holds n_list * q_heads * max_splits * (head_dim + 2) floats.
TIE_API int tie_attention_split(int dtype, const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                void* out, const int* query_start, const int* context_lens, const int* block_tables,
                                int max_blocks, int seqs, int q_heads, int kv_heads, int head_dim, int page_size,
                                int window, float scale, const int* seq_list, int n_list, int split_keys,
                                int max_splits, float* scratch, cudaStream_t s) {
  const AttnArgs a{q, k_cache, v_cache, out, nullptr, query_start, context_lens, block_tables, q_stride, max_blocks,
                   0, seqs, q_heads, kv_heads, head_dim, page_size, window, scale, head_dim};
  if (const int st = check_attn(a)) return st;
  TIE_REQUIRE(split_keys > 0 && max_splits > 0 && max_splits <= kMergeMaxSplits && scratch != nullptr,
              "attention split: bad split geometry (at most %d splits)", kMergeMaxSplits);
  if (dtype == TIE_F32) return launch_attention<float>(a, nullptr, seq_list, n_list, split_keys, max_splits, scratch, 0, s);
  if (dtype == TIE_BF16)
    return launch_attention<__nv_bfloat16>(a, nullptr, seq_list, n_list, split_keys, max_splits, scratch, 0, s);
  set_error("attention: unknown dtype code %d", dtype);
  return kBadArgument;
}

// Combines the (acc, max, sum) that a split kernel (this file's or the tensor-core one) left in
// scratch [n_list, q_heads, max_splits, head_dim + 2] into out rows, in split order.
TIE_API int tie_attention_merge(int dtype, void* out, const int* query_start, const int* context_lens, int q_heads,
                                int head_dim, int window, const int* seq_list, int n_list, int split_keys, int max_splits,
                                const float* scratch, cudaStream_t s) {
  TIE_REQUIRE(q_heads > 0 && head_dim > 0 && split_keys > 0 && max_splits > 0 && max_splits <= kMergeMaxSplits,
              "attention merge: bad geometry (at most %d splits)", kMergeMaxSplits);
  if (n_list == 0) return kOk;
  AttnArgs a{};
  a.out = out;
  a.query_start = query_start;
  a.context_lens = context_lens;
  a.q_heads = q_heads;
  a.head_dim = head_dim;
  a.window = window;
  const long long items = static_cast<long long>(n_list) * q_heads;
  if (dtype == TIE_F32) {
    TIE_LAUNCH((attention_merge_kernel<float>), static_cast<int>(items), kMergeThreads, 0, s, a, seq_list, n_list, split_keys, max_splits, scratch);
  } else if (dtype == TIE_BF16) {
    TIE_LAUNCH((attention_merge_kernel<__nv_bfloat16>), static_cast<int>(items), kMergeThreads, 0, s, a, seq_list, n_list, split_keys, max_splits, scratch);
  } else {
    set_error("attention merge: unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("attention_merge");
}

// The same two for keys and values of different head sizes: queries and keys have head_dim, values and the
// output v_dim (planes [pages, kv_heads, page_size, head_dim] and [pages, kv_heads, page_size, v_dim]).
TIE_API int tie_attention_rows_dv(int dtype, const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                  void* out, const int* seq_of_row, const int* query_start, const int* context_lens,
                                  const int* block_tables, int max_blocks, int rows, int seqs, int q_heads, int kv_heads,
                                  int head_dim, int v_dim, int page_size, int window, float scale, int v_ld,
                                  cudaStream_t s) {
  const AttnArgs a{q, k_cache, v_cache, out, seq_of_row, query_start, context_lens, block_tables, q_stride, max_blocks,
                   rows, seqs, q_heads, kv_heads, head_dim, page_size, window, scale, v_dim, v_ld};
  TIE_REQUIRE(v_ld == 0 || v_ld >= v_dim, "attention: value rows %d apart are shorter than a value head of %d", v_ld, v_dim);
  if (const int st = check_attn(a, true)) return st;
  if (dtype == TIE_F32) return launch_attention<float>(a, nullptr, nullptr, 0, 0, 0, nullptr, 1, s);
  if (dtype == TIE_BF16) return launch_attention<__nv_bfloat16>(a, nullptr, nullptr, 0, 0, 0, nullptr, 1, s);
  set_error("attention: unknown dtype code %d", dtype);
  return kBadArgument;
}

TIE_API int tie_attention_split_dv(int dtype, const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                   void* out, const int* query_start, const int* context_lens, const int* block_tables,
                                   int max_blocks, int seqs, int q_heads, int kv_heads, int head_dim, int v_dim,
                                   int page_size, int window, float scale, const int* seq_list, int n_list, int split_keys,
                                   int max_splits, float* scratch, int v_ld, cudaStream_t s) {
  const AttnArgs a{q, k_cache, v_cache, out, nullptr, query_start, context_lens, block_tables, q_stride, max_blocks,
                   0, seqs, q_heads, kv_heads, head_dim, page_size, window, scale, v_dim, v_ld};
  TIE_REQUIRE(v_ld == 0 || v_ld >= v_dim, "attention: value rows %d apart are shorter than a value head of %d", v_ld, v_dim);
  if (const int st = check_attn(a, true)) return st;
  TIE_REQUIRE(split_keys > 0 && max_splits > 0 && max_splits <= kMergeMaxSplits && scratch != nullptr,
              "attention split: bad split geometry (at most %d splits)", kMergeMaxSplits);
  if (dtype == TIE_F32) return launch_attention<float>(a, nullptr, seq_list, n_list, split_keys, max_splits, scratch, 0, s);
  if (dtype == TIE_BF16)
    return launch_attention<__nv_bfloat16>(a, nullptr, seq_list, n_list, split_keys, max_splits, scratch, 0, s);
  set_error("attention: unknown dtype code %d", dtype);
  return kBadArgument;
}

// Score maps over slices of wider key rows (the fields of AttnArgs behind v_ld): the planes are
// [pages, kv_heads, page_size, k_ld] and [pages, kv_heads, page_size, v_dim]; query head h reads kv head
// (h / group) % kv_heads and, of its key row, the head_dim elements from ((h / sub_div) % sub_count) * head_dim;
// its softmax weights meet the whole value row. Chunks, a cap on the scores and a bias by the logarithm of the
// distance are options. The output rows [T, q_heads * v_dim] are float.
TIE_API int tie_attention_maps_rows(int dtype, const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                    float* out, const int* seq_of_row, const int* query_start, const int* context_lens,
                                    const int* block_tables, int max_blocks, int rows, int seqs, int q_heads, int kv_heads,
                                    int head_dim, int k_ld, int sub_div, int sub_count, int v_dim, int page_size, int window,
                                    int chunk, float scale, float softcap, const float* r1, const float* r2, int group,
                                    cudaStream_t s) {
  const AttnArgs a{q, k_cache, v_cache, out, seq_of_row, query_start, context_lens, block_tables, q_stride, max_blocks,
                   rows, seqs, q_heads, kv_heads, head_dim, page_size, window, scale, v_dim, 0, k_ld, sub_div, sub_count,
                   chunk, softcap, r1, r2, 1, group};
  TIE_REQUIRE(group > 0, "attention maps: query heads per cached head must be positive");
  TIE_REQUIRE(sub_div > 0 && sub_count > 0 && k_ld >= sub_count * head_dim && chunk >= 0 && (r1 == nullptr) == (r2 == nullptr),
              "attention maps: %d slices of %d do not fit key rows of %d", sub_count, head_dim, k_ld);
  if (const int st = check_attn(a, true)) return st;
  if (dtype == TIE_F32) return launch_attention<float>(a, nullptr, nullptr, 0, 0, 0, nullptr, 1, s);
  if (dtype == TIE_BF16) return launch_attention<__nv_bfloat16>(a, nullptr, nullptr, 0, 0, 0, nullptr, 1, s);
  set_error("attention: unknown dtype code %d", dtype);
  return kBadArgument;
}

TIE_API int tie_attention_maps_split(int dtype, const void* q, long long q_stride, const void* k_cache, const void* v_cache,
                                     float* out, const int* query_start, const int* context_lens, const int* block_tables,
                                     int max_blocks, int seqs, int q_heads, int kv_heads, int head_dim, int k_ld, int sub_div,
                                     int sub_count, int v_dim, int page_size, int window, int chunk, float scale, float softcap,
                                     const float* r1, const float* r2, int group, const int* seq_list, int n_list, int split_keys,
                                     int max_splits, float* scratch, cudaStream_t s) {
  const AttnArgs a{q, k_cache, v_cache, out, nullptr, query_start, context_lens, block_tables, q_stride, max_blocks,
                   0, seqs, q_heads, kv_heads, head_dim, page_size, window, scale, v_dim, 0, k_ld, sub_div, sub_count,
                   chunk, softcap, r1, r2, 1, group};
  TIE_REQUIRE(group > 0, "attention maps: query heads per cached head must be positive");
  TIE_REQUIRE(sub_div > 0 && sub_count > 0 && k_ld >= sub_count * head_dim && chunk >= 0 && (r1 == nullptr) == (r2 == nullptr),
              "attention maps: %d slices of %d do not fit key rows of %d", sub_count, head_dim, k_ld);
  if (const int st = check_attn(a, true)) return st;
  TIE_REQUIRE(split_keys > 0 && max_splits > 0 && max_splits <= kMergeMaxSplits && scratch != nullptr,
              "attention split: bad split geometry (at most %d splits)", kMergeMaxSplits);
  if (dtype == TIE_F32) return launch_attention<float>(a, nullptr, seq_list, n_list, split_keys, max_splits, scratch, 0, s, true);
  if (dtype == TIE_BF16)
    return launch_attention<__nv_bfloat16>(a, nullptr, seq_list, n_list, split_keys, max_splits, scratch, 0, s, true);
  set_error("attention: unknown dtype code %d", dtype);
  return kBadArgument;
}

// ---------------------------------------------------------------------------------------------
// The variant of tie_attention_split that allocates nothing (see attention_noalloc.h).
#include "attention_noalloc.h"

namespace tie {
// Partial results of the splits. In host code this name is only a handle for
// cudaGetSymbolAddress; the address a kernel can use is looked up once per device below.
static __device__ __align__(256) float g_noalloc_scratch[TIE_NOALLOC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
static float* g_noalloc_ptr[kMaxDevices] = {};   // device address of the array on each device, once known
}  // namespace tie

TIE_API int tie_attention_split_noalloc(int dtype, const void* q, long long q_stride, const void* k_cache,
                                        const void* v_cache, void* out, const int* query_start, const int* context_lens,
                                        const int* block_tables, int max_blocks, int seqs, int q_heads, int kv_heads,
                                        int head_dim, int page_size, int window, float scale, const int* seq_list,
                                        int n_list, int split_keys, int max_splits, cudaStream_t s) {
  const AttnArgs a{q, k_cache, v_cache, out, nullptr, query_start, context_lens, block_tables, q_stride, max_blocks,
                   0, seqs, q_heads, kv_heads, head_dim, page_size, window, scale, head_dim};
  if (const int st = check_attn(a)) return st;
  TIE_REQUIRE(n_list >= 0 && split_keys > 0 && max_splits > 0 && max_splits <= kMergeMaxSplits,
              "attention split (no alloc): bad split geometry (at most %d splits)", kMergeMaxSplits);
  const long long need = static_cast<long long>(n_list) * q_heads * max_splits * (head_dim + 2);
  TIE_REQUIRE(need <= TIE_NOALLOC_SCRATCH_FLOATS,
              "attention split (no alloc): %d sequences x %d heads x %d splits x (%d + 2) = %lld floats of partial results "
              "exceed the built-in %d; use fewer splits or tie_attention_split with your own scratch",
              n_list, q_heads, max_splits, head_dim, need, TIE_NOALLOC_SCRATCH_FLOATS);
  int device = -1;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) {
    set_error("attention split (no alloc): cannot use device %d (at most %d devices)", device, kMaxDevices);
    return kCudaError;
  }
  if (g_noalloc_ptr[device] == nullptr) {   // set-up, once per device, with that device current
    float* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_error("attention split (no alloc): cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return kCudaError;
    }
    g_noalloc_ptr[device] = p;
  }
  float* scratch = g_noalloc_ptr[device];
  if (dtype == TIE_F32) return launch_attention<float>(a, nullptr, seq_list, n_list, split_keys, max_splits, scratch, 0, s);
  if (dtype == TIE_BF16)
    return launch_attention<__nv_bfloat16>(a, nullptr, seq_list, n_list, split_keys, max_splits, scratch, 0, s);
  set_error("attention: unknown dtype code %d", dtype);
  return kBadArgument;
}
