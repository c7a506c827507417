// Kernels of a layer whose two sublayers read the same stream side by side, and of what such models put around it:
//
//   pair_hash_add     x[t] += table[row], row = (prev * mul_prev + token * mul_cur) mod buckets for the pair (previous
//                     token, token), or the table's last row for a sequence's first token. The previous token of a
//                     portion's first row comes from the request's state slot; the block of that row also stores the
//                     portion's last token there (no other block touches the slot).
//   add_row_vector    x[t] += vec for every row (one learned vector ahead of a pass over a span of layers).
//   group_norm_taps   u = x / rms over each of `groups` equal parts of the row (float). Outputs, one per sublayer:
//                     out_a = w_a * (u_t + sum_j taps_a[j] * u_(t - taps + 1 + j)) (taps_a [taps, D]: a tap of every
//                     channel side by side, for coalesced reads), that is h + conv(h) for h = u * w_a,
//                     a causal convolution over time per channel with zeros ahead of the sequence. Rows of this step
//                     are renormed from x (x is complete when the kernel starts); rows of earlier steps come from the
//                     request's state, a ring of the last taps - 1 unit rows indexed by position. The rows that will
//                     be that ring after the step are left in `unit`; parallel_finish moves them (it runs when every
//                     block here has read the ring). With taps = 0 it is a plain grouped norm, optionally over
//                     gathered rows and with a delta added to x first.
//   parallel_finish   x += mult * (delta_a + delta_b) (tensors or float partial sums, added in order), then the token
//                     side input: g = gelu_tanh(W_gate x) * table[token], y = W_proj g, x += mult * y / rms(y) * w;
//                     then the ring update. Sums, norms and the stream in float.
//   For many rows the side input's two products run as matrix products instead, between three small kernels:
//   parallel_sum      x += mult * (delta_a + delta_b); copy = x in the storage type (the first product's input).
//   side_gate_act     g = gelu_tanh(pre) * table[token] for pre = copy W_gate^T (float), in the storage type.
//   side_finish       x += mult * y / rms(y) * w for y = g W_proj^T (float), then the ring update.
#include <math.h>

#include "common.cuh"

namespace tie {

template <typename T>
__global__ void __launch_bounds__(128) pair_hash_add_kernel(float* __restrict__ x, const T* __restrict__ table,
                                                            const int* __restrict__ tokens, const int* __restrict__ positions,
                                                            const int* __restrict__ seq_of_row, const int* __restrict__ query_start,
                                                            const int* __restrict__ state_slots, int* __restrict__ prev_state,
                                                            int buckets, long long mul_prev, long long mul_cur, int dim) {
  pdl_sync();
  __shared__ int srow;
  const int t = blockIdx.x;
  if (threadIdx.x == 0) {
    const int s = seq_of_row[t], pos = positions[t], q0 = query_start[s];
    const int slot = state_slots[s];
    int row = buckets;
    if (pos > 0) {
      const long long prev = t > q0 ? tokens[t - 1] : (slot >= 0 ? prev_state[slot] : 0);
      long long r = (prev * mul_prev + static_cast<long long>(tokens[t]) * mul_cur) % buckets;
      if (r < 0) r += buckets;
      row = static_cast<int>(r);
    }
    srow = row;
    if (t == q0 && slot >= 0) prev_state[slot] = tokens[query_start[s + 1] - 1];
  }
  __syncthreads();
  const T* src = table + static_cast<long long>(srow) * dim;
  float* xr = x + static_cast<long long>(t) * dim;
  for (int d = threadIdx.x; d < dim; d += blockDim.x) xr[d] += ld(src + d);
}

__global__ void __launch_bounds__(256) add_row_vector_kernel(float* __restrict__ x, const float* __restrict__ vec, int dim,
                                                             long long total) {
  pdl_sync();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < total) x[i] += vec[i % dim];
}

constexpr int kMaxTaps = 8;

struct Delta {            // what a sublayer hands on: a tensor in the storage type, or float partial sums, or nothing
  const void* tensor;
  const float* part;
  long long part_stride;
  int splits;
};

template <typename T>
__device__ __forceinline__ float delta_at(const Delta& d, long long idx) {
  if (d.tensor != nullptr) return ld(static_cast<const T*>(d.tensor) + idx);
  float y = 0.0f;
  if (d.part != nullptr)
    for (int z = 0; z < d.splits; ++z) y += d.part[z * d.part_stride + idx];
  return y;
}

struct NormTapsArgs {
  float* x;                 // [T, D]
  Delta delta;              // taps == 0 only: added to x first (written back unless rows are gathered)
  const int* rows;          // taps == 0 only: output row i reads row rows[i] (null: i)
  int n, D, groups;
  float eps;
  const float* w_a;
  const float* w_b;         // null: one output
  const float* taps_a;      // [taps, D] float (null with taps == 0)
  const float* taps_b;
  int taps;
  void* out_a;
  void* out_b;
  float* unit;              // [T, D]
  const float* ring;        // [slots, taps - 1, D]
  const int* seq_of_row;
  const int* positions;
  const int* query_start;
  const int* context_lens;
  const int* state_slots;
};

// The grouped norm alone (no taps): optionally a delta added to x first, optionally gathered rows. A block a row.
template <typename T>
__global__ void __launch_bounds__(256) group_norm_taps_kernel(NormTapsArgs a) {
  pdl_sync();
  extern __shared__ float smem[];
  float* inv = smem;                       // [groups]
  const int i = blockIdx.x;
  const int t = a.rows != nullptr ? a.rows[i] : i;
  const int D = a.D;
  const int gsize = D / a.groups;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  float* xr = a.x + static_cast<long long>(t) * D;
  if (a.delta.tensor != nullptr || a.delta.part != nullptr) {
    float* row = smem + a.groups;          // the summed row, kept for both passes
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      const float v = xr[d] + delta_at<T>(a.delta, static_cast<long long>(t) * D + d);
      row[d] = v;
      if (a.rows == nullptr) xr[d] = v;
    }
    __syncthreads();
    xr = row;
  }
  for (int g = warp; g < a.groups; g += nwarps) {
    const float* src = xr + g * gsize;
    float ss = 0.0f;
    for (int d = lane; d < gsize; d += 32) ss = fmaf(src[d], src[d], ss);
    ss = warp_sum(ss);
    if (lane == 0) inv[g] = 1.0f / sqrtf(ss / static_cast<float>(gsize) + a.eps);
  }
  __syncthreads();
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float u = xr[d] * inv[d / gsize];
    st(static_cast<T*>(a.out_a) + static_cast<long long>(i) * D + d, a.w_a[d] * u);
    if (a.w_b != nullptr) st(static_cast<T*>(a.out_b) + static_cast<long long>(i) * D + d, a.w_b[d] * u);
  }
}

__device__ __forceinline__ void store_vec(float* p, const float (&v)[4]) { *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]); }
__device__ __forceinline__ void store_vec(__nv_bfloat16* p, const float (&v)[4]) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<const uint32_t*>(&lo), *reinterpret_cast<const uint32_t*>(&hi));
}
__device__ __forceinline__ void store_vec(float* p, const float (&v)[1]) { p[0] = v[0]; }
__device__ __forceinline__ void store_vec(__nv_bfloat16* p, const float (&v)[1]) { st(p, v[0]); }
template <int W> __device__ __forceinline__ void load_vec(const float* p, float (&v)[W]) {
  if constexpr (W == 4) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    v[0] = t.x, v[1] = t.y, v[2] = t.z, v[3] = t.w;
  } else {
    v[0] = p[0];
  }
}

// group_norm_taps with TAPS taps for `tile` consecutive rows a block: the norms of the tile's rows and of the TAPS - 1
// rows before it are computed once (a warp per row and group); then a thread owns W columns and walks down the tile's
// rows with the unit values of the TAPS - 1 rows above in registers, so that x is read once a tile (plus the rows
// above it) and the tap weights once a thread. A row whose predecessors are not in this step (another sequence above
// it, or an earlier step) takes them from its request's ring, or zeros ahead of position 0. A row's numbers do not
// depend on the tile it falls into.
template <typename T, int W, int TAPS>
__global__ void __launch_bounds__(256) group_norm_taps_tile_kernel(NormTapsArgs a, int tile) {
  pdl_sync();
  extern __shared__ float smem[];
  constexpr int R = TAPS - 1, RR = R > 0 ? R : 1;
  float* inv = smem;                       // [(tile + R) * groups], row t0 - R first
  const int D = a.D, G = a.groups;
  const int gsize = D / G;
  const int t0 = blockIdx.x * tile;
  const int nr = min(tile, a.n - t0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int item = warp; item < (nr + R) * G; item += nwarps) {
    const int j = item / G, g = item - j * G;
    const int t = t0 - R + j;
    if (t < 0) continue;
    const float* src = a.x + static_cast<long long>(t) * D + g * gsize;
    float ss = 0.0f;
    for (int d = lane * W; d < gsize; d += 32 * W) {
      float v[W];
      load_vec<W>(src + d, v);
#pragma unroll
      for (int e = 0; e < W; ++e) ss = fmaf(v[e], v[e], ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) inv[item] = 1.0f / sqrtf(ss / static_cast<float>(gsize) + a.eps);
  }
  int* meta = reinterpret_cast<int*>(inv + (tile + R) * G);      // [tile][4]: position, the portion's first position, slot, keep
  for (int j = threadIdx.x; j < nr; j += blockDim.x) {
    const int t = t0 + j;
    const int s = a.seq_of_row[t];
    const int pos = a.positions[t];
    meta[4 * j] = pos;
    meta[4 * j + 1] = pos - (t - a.query_start[s]);
    meta[4 * j + 2] = a.state_slots[s];
    meta[4 * j + 3] = R > 0 && pos >= a.context_lens[s] - R;
  }
  __syncthreads();
  const bool two = a.w_b != nullptr;
  for (int d = threadIdx.x * W; d < D; d += blockDim.x * W) {
    const int g = d / gsize;
    float wa[TAPS][W], wb[TAPS][W], na[W], nb[W];
#pragma unroll
    for (int k = 0; k < TAPS; ++k) {
      load_vec<W>(a.taps_a + static_cast<long long>(k) * D + d, wa[k]);
      if (two) load_vec<W>(a.taps_b + static_cast<long long>(k) * D + d, wb[k]);
    }
    load_vec<W>(a.w_a + d, na);
    if (two) load_vec<W>(a.w_b + d, nb);
    float win[RR][W];                      // win[r - 1]: the unit value of the row r above the current one
#pragma unroll
    for (int r = 1; r <= R; ++r) {
#pragma unroll
      for (int e = 0; e < W; ++e) win[r - 1][e] = 0.0f;
      if (t0 - r >= 0) {
        load_vec<W>(a.x + static_cast<long long>(t0 - r) * D + d, win[r - 1]);
        const float scale = inv[(R - r) * G + g];
#pragma unroll
        for (int e = 0; e < W; ++e) win[r - 1][e] *= scale;
      }
    }
    for (int j = 0; j < nr; ++j) {
      const int t = t0 + j;
      const int pos = meta[4 * j], first = meta[4 * j + 1], slot = meta[4 * j + 2];
      float u[TAPS][W];
      load_vec<W>(a.x + static_cast<long long>(t) * D + d, u[0]);
      const float scale = inv[(j + R) * G + g];
#pragma unroll
      for (int e = 0; e < W; ++e) u[0][e] *= scale;
#pragma unroll
      for (int r = 1; r <= R; ++r) {
        const int p = pos - r;
        if (p >= first) {
#pragma unroll
          for (int e = 0; e < W; ++e) u[r][e] = win[r - 1][e];
        } else if (p >= 0 && slot >= 0) {
          load_vec<W>(a.ring + (static_cast<long long>(slot) * R + p % RR) * D + d, u[r]);
        } else {
#pragma unroll
          for (int e = 0; e < W; ++e) u[r][e] = 0.0f;
        }
      }
      float oa[W], ob[W];
#pragma unroll
      for (int e = 0; e < W; ++e) oa[e] = ob[e] = u[0][e];
#pragma unroll
      for (int r = R; r >= 0; --r) {       // tap TAPS - 1 - r reads the row r back; the oldest row first
#pragma unroll
        for (int e = 0; e < W; ++e) {
          oa[e] = fmaf(wa[R - r][e], u[r][e], oa[e]);
          if (two) ob[e] = fmaf(wb[R - r][e], u[r][e], ob[e]);
        }
      }
#pragma unroll
      for (int e = 0; e < W; ++e) oa[e] *= na[e];
      store_vec(static_cast<T*>(a.out_a) + static_cast<long long>(t) * D + d, oa);
      if (two) {
#pragma unroll
        for (int e = 0; e < W; ++e) ob[e] *= nb[e];
        store_vec(static_cast<T*>(a.out_b) + static_cast<long long>(t) * D + d, ob);
      }
      if (meta[4 * j + 3] != 0) store_vec(a.unit + static_cast<long long>(t) * D + d, u[0]);
#pragma unroll
      for (int r = R; r >= 2; --r) {
#pragma unroll
        for (int e = 0; e < W; ++e) win[r - 1][e] = win[r - 2][e];
      }
      if (R > 0) {
#pragma unroll
        for (int e = 0; e < W; ++e) win[0][e] = u[0][e];
      }
    }
  }
}

__device__ __forceinline__ float gelu_tanh_side(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

struct FinishArgs {
  float* x;
  int T, D;
  float mult;
  Delta a, b;
  // token side input (side_dim == 0: none)
  const int* tokens;
  const void* side_table;      // [vocab, side_dim] in the storage type
  const void* side_gate;       // [side_dim, D]
  const void* side_proj;       // [D, side_dim]
  const float* side_norm;      // [D]
  int side_dim;
  float eps;
  // ring of unit rows (R == 0: none)
  const float* unit;
  float* ring;
  int R;
  const int* seq_of_row;
  const int* positions;
  const int* context_lens;
  const int* state_slots;
};

// RB rows a block (one, as launched: steps of many rows take the side input as matrix products instead).
template <typename T, int RB>
__global__ void __launch_bounds__(256) parallel_finish_kernel(FinishArgs a) {
  pdl_sync();
  extern __shared__ float smem[];
  const int D = a.D, S = a.side_dim;
  float* row = smem;                   // [RB][D]: the summed rows, later the side input's y
  float* g = row + RB * D;             // [RB][S]
  float* scratch = g + RB * S;         // [33]
  const int t0 = blockIdx.x * RB;
  const int nr = min(RB, a.T - t0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  constexpr int V = Vec16<T>::N;
  for (int r = 0; r < nr; ++r) {
    float* xr = a.x + static_cast<long long>(t0 + r) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      const long long idx = static_cast<long long>(t0 + r) * D + d;
      const float v = xr[d] + a.mult * (delta_at<T>(a.a, idx) + delta_at<T>(a.b, idx));
      row[r * D + d] = v;
      xr[d] = v;
    }
  }
  if (S > 0) {
    __syncthreads();
    const T* gate = static_cast<const T*>(a.side_gate);
    const T* table = static_cast<const T*>(a.side_table);
    const bool wide_d = D % V == 0, wide_s = S % V == 0;
    for (int i = warp; i < S; i += nwarps) {
      const T* wr = gate + static_cast<long long>(i) * D;
      float dot[RB];
#pragma unroll
      for (int r = 0; r < RB; ++r) dot[r] = 0.0f;
      if (wide_d) {
        for (int d = lane * V; d < D; d += 32 * V) {
          Vec16<T> w;
          w.load(wr + d);
#pragma unroll
          for (int r = 0; r < RB; ++r) {
            if (r < nr) {
#pragma unroll
              for (int e = 0; e < V; ++e) dot[r] = fmaf(w.v[e], row[r * D + d + e], dot[r]);
            }
          }
        }
      } else {
        for (int d = lane; d < D; d += 32) {
          const float w = ld(wr + d);
#pragma unroll
          for (int r = 0; r < RB; ++r)
            if (r < nr) dot[r] = fmaf(w, row[r * D + d], dot[r]);
        }
      }
#pragma unroll
      for (int r = 0; r < RB; ++r) {
        const float sum = warp_sum(dot[r]);
        if (lane == 0 && r < nr) g[r * S + i] = gelu_tanh_side(sum) * ld(table + static_cast<long long>(a.tokens[t0 + r]) * S + i);
      }
    }
    __syncthreads();
    const T* proj = static_cast<const T*>(a.side_proj);
    float ss[RB];
#pragma unroll
    for (int r = 0; r < RB; ++r) ss[r] = 0.0f;
    for (int d = threadIdx.x; d < D; d += blockDim.x) {
      const T* wr = proj + static_cast<long long>(d) * S;
      float y[RB];
#pragma unroll
      for (int r = 0; r < RB; ++r) y[r] = 0.0f;
      if (wide_s) {
        for (int i = 0; i < S; i += V) {
          Vec16<T> w;
          w.load(wr + i);
#pragma unroll
          for (int r = 0; r < RB; ++r) {
            if (r < nr) {
#pragma unroll
              for (int e = 0; e < V; ++e) y[r] = fmaf(w.v[e], g[r * S + i + e], y[r]);
            }
          }
        }
      } else {
        for (int i = 0; i < S; ++i) {
          const float w = ld(wr + i);
#pragma unroll
          for (int r = 0; r < RB; ++r)
            if (r < nr) y[r] = fmaf(w, g[r * S + i], y[r]);
        }
      }
#pragma unroll
      for (int r = 0; r < RB; ++r) {
        if (r < nr) {
          ss[r] = fmaf(y[r], y[r], ss[r]);
          row[r * D + d] = y[r];        // this thread's own column: the summed row is in x already
        }
      }
    }
#pragma unroll
    for (int r = 0; r < RB; ++r) {
      const float total = block_sum(ss[r], scratch);
      if (r < nr) {
        const float inv = 1.0f / sqrtf(total / static_cast<float>(D) + a.eps);
        float* xr = a.x + static_cast<long long>(t0 + r) * D;
        for (int d = threadIdx.x; d < D; d += blockDim.x) xr[d] += a.mult * (row[r * D + d] * inv) * a.side_norm[d];
      }
    }
  }
  if (a.R > 0) {
    for (int r = 0; r < nr; ++r) {
      const int t = t0 + r;
      const int s = a.seq_of_row[t];
      const int pos = a.positions[t], slot = a.state_slots[s];
      if (slot >= 0 && pos >= a.context_lens[s] - a.R) {
        const float* src = a.unit + static_cast<long long>(t) * D;
        float* dst = a.ring + (static_cast<long long>(slot) * a.R + pos % a.R) * D;
        for (int d = threadIdx.x; d < D; d += blockDim.x) dst[d] = src[d];
      }
    }
  }
}

// parallel_finish for few rows: a row is shared by the kFinishCluster CTAs of a thread-block cluster, so that a decode
// step of a handful of rows still reads the side input's weights with dozens of CTAs. Every CTA forms the whole summed
// row (the gate's products need all of it) and owns a slice of the gate's outputs and a slice of the columns: the
// slices of g are gathered, and the parts of sum(y^2) added in rank order, through distributed shared memory.
constexpr int kFinishCluster = 8;

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ float peer_shared_float(const float* mine, uint32_t rank) {
  uint32_t addr;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"(static_cast<uint32_t>(__cvta_generic_to_shared(mine))), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

template <typename T>
__global__ void __launch_bounds__(256) parallel_finish_cluster_kernel(FinishArgs a) {
  pdl_sync();
  extern __shared__ float smem[];
  const int D = a.D, S = a.side_dim;
  constexpr int C = kFinishCluster, V = Vec16<T>::N;
  float* row = smem;                   // [D]: the summed row; this CTA's columns later hold y
  float* g = row + D;                  // [S]
  float* scratch = g + S;              // [33]
  float* part = scratch + 36;          // this CTA's part of sum(y^2)
  const int rank = static_cast<int>(cluster_rank());
  const int t = blockIdx.x / C;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const int cols = ((D + C - 1) / C + V - 1) / V * V;          // columns a CTA, whole 16-byte pieces
  const int d_lo = min(D, rank * cols), d_hi = min(D, d_lo + cols);
  const int outs = (S + C - 1) / C;
  const int i_lo = min(S, rank * outs), i_hi = min(S, i_lo + outs);
  float* xr = a.x + static_cast<long long>(t) * D;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const long long idx = static_cast<long long>(t) * D + d;
    const float v = xr[d] + a.mult * (delta_at<T>(a.a, idx) + delta_at<T>(a.b, idx));
    row[d] = v;               // x itself is written after the cluster's first barrier: until then the peers read it
  }
  __syncthreads();
  {
    const T* gate = static_cast<const T*>(a.side_gate);
    const T* table = static_cast<const T*>(a.side_table) + static_cast<long long>(a.tokens[t]) * S;
    const bool wide = D % V == 0;
    for (int i = i_lo + warp; i < i_hi; i += nwarps) {
      const T* wr = gate + static_cast<long long>(i) * D;
      float dot = 0.0f;
      if (wide) {
        for (int d = lane * V; d < D; d += 32 * V) {
          Vec16<T> w;
          w.load(wr + d);
#pragma unroll
          for (int e = 0; e < V; ++e) dot = fmaf(w.v[e], row[d + e], dot);
        }
      } else {
        for (int d = lane; d < D; d += 32) dot = fmaf(ld(wr + d), row[d], dot);
      }
      dot = warp_sum(dot);
      if (lane == 0) g[i] = gelu_tanh_side(dot) * ld(table + i);
    }
  }
  cluster_sync_all();                  // every CTA's slice of g is written, and every CTA has read the row of x
  for (int d = d_lo + threadIdx.x; d < d_hi; d += blockDim.x) xr[d] = row[d];
  for (int i = threadIdx.x; i < S; i += blockDim.x) {
    const int owner = i / outs;
    if (owner != rank) g[i] = peer_shared_float(g + i, owner);
  }
  __syncthreads();
  float ss = 0.0f;
  {
    const T* proj = static_cast<const T*>(a.side_proj);
    const bool wide = S % V == 0;
    for (int d = d_lo + threadIdx.x; d < d_hi; d += blockDim.x) {
      const T* wr = proj + static_cast<long long>(d) * S;
      float y = 0.0f;
      if (wide) {
        for (int i = 0; i < S; i += V) {
          Vec16<T> w;
          w.load(wr + i);
#pragma unroll
          for (int e = 0; e < V; ++e) y = fmaf(w.v[e], g[i + e], y);
        }
      } else {
        for (int i = 0; i < S; ++i) y = fmaf(ld(wr + i), g[i], y);
      }
      ss = fmaf(y, y, ss);
      row[d] = y;
    }
  }
  ss = block_sum(ss, scratch);
  if (threadIdx.x == 0) *part = ss;
  cluster_sync_all();                  // every CTA's part is written (and nobody reads a peer's g any more)
  float total = 0.0f;
  for (int r = 0; r < C; ++r) total += r == rank ? ss : peer_shared_float(part, r);
  const float inv = 1.0f / sqrtf(total / static_cast<float>(D) + a.eps);
  for (int d = d_lo + threadIdx.x; d < d_hi; d += blockDim.x) xr[d] += a.mult * (row[d] * inv) * a.side_norm[d];
  if (a.R > 0) {
    const int s = a.seq_of_row[t];
    const int pos = a.positions[t], slot = a.state_slots[s];
    if (slot >= 0 && pos >= a.context_lens[s] - a.R) {
      const float* src = a.unit + static_cast<long long>(t) * D;
      float* dst = a.ring + (static_cast<long long>(slot) * a.R + pos % a.R) * D;
      for (int d = d_lo + threadIdx.x; d < d_hi; d += blockDim.x) dst[d] = src[d];
    }
  }
  cluster_sync_all();                  // a CTA's shared memory stays until every peer has read its part
}

template <typename T>
static int launch_finish_cluster(const FinishArgs& a, cudaStream_t s) {
  const size_t smem = (static_cast<size_t>(a.D) + a.side_dim + 48) * sizeof(float);
  if (smem > 48 * 1024) cudaFuncSetAttribute(parallel_finish_cluster_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(a.T * kFinishCluster);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = kFinishCluster;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = pdl_enabled() ? 2 : 1;
  cudaLaunchKernelEx(&cfg, parallel_finish_cluster_kernel<T>, a);
  TIE_RETURN_LAUNCH("parallel_finish");
}

// Four consecutive elements of a delta (idx a multiple of 4, the row width too).
__device__ __forceinline__ void load4_as_float(const float* p, float (&v)[4]) { load_vec<4>(p, v); }
__device__ __forceinline__ void load4_as_float(const __nv_bfloat16* p, float (&v)[4]) {
  const uint2 t = *reinterpret_cast<const uint2*>(p);
  v[0] = __uint_as_float(t.x << 16), v[1] = __uint_as_float(t.x & 0xffff0000u);
  v[2] = __uint_as_float(t.y << 16), v[3] = __uint_as_float(t.y & 0xffff0000u);
}
template <typename T>
__device__ __forceinline__ void delta_at4(const Delta& d, long long idx, float (&y)[4]) {
  y[0] = y[1] = y[2] = y[3] = 0.0f;
  if (d.tensor != nullptr) {
    load4_as_float(static_cast<const T*>(d.tensor) + idx, y);
  } else if (d.part != nullptr) {
    for (int z = 0; z < d.splits; ++z) {
      float p[4];
      load_vec<4>(d.part + z * d.part_stride + idx, p);
#pragma unroll
      for (int e = 0; e < 4; ++e) y[e] += p[e];
    }
  }
}

// W = 4: four columns a thread (the row width and, with partial sums, their stride are multiples of 4).
template <typename T, int W>
__global__ void __launch_bounds__(256) parallel_sum_kernel(float* __restrict__ x, T* __restrict__ copy, int D, float mult, Delta da, Delta db) {
  pdl_sync();
  const long long base = static_cast<long long>(blockIdx.x) * D;
  for (int d = threadIdx.x * W; d < D; d += blockDim.x * W) {
    float v[W];
    if constexpr (W == 4) {
      float a[4], b[4];
      load_vec<4>(x + base + d, v);
      delta_at4<T>(da, base + d, a);
      delta_at4<T>(db, base + d, b);
#pragma unroll
      for (int e = 0; e < 4; ++e) v[e] += mult * (a[e] + b[e]);
    } else {
      v[0] = x[base + d] + mult * (delta_at<T>(da, base + d) + delta_at<T>(db, base + d));
    }
    store_vec(x + base + d, v);
    store_vec(copy + base + d, v);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) side_gate_act_kernel(const float* __restrict__ pre, const T* __restrict__ table,
                                                            const int* __restrict__ tokens, T* __restrict__ g, int S, long long total) {
  pdl_sync();
  const long long e = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (e >= total) return;
  const long long t = e / S;
  const int i = static_cast<int>(e - t * S);
  st(g + e, gelu_tanh_side(pre[e]) * ld(table + static_cast<long long>(tokens[t]) * S + i));
}

struct SideFinishArgs {
  float* x;
  const float* y;
  int D;
  float mult, eps;
  const float* w;
  const float* unit;
  float* ring;
  int R;
  const int* seq_of_row;
  const int* positions;
  const int* context_lens;
  const int* state_slots;
};

template <int W>
__global__ void __launch_bounds__(256) side_finish_kernel(SideFinishArgs a) {
  pdl_sync();
  __shared__ float scratch[40];
  const int t = blockIdx.x, D = a.D;
  const float* yr = a.y + static_cast<long long>(t) * D;
  float* xr = a.x + static_cast<long long>(t) * D;
  float ss = 0.0f;
  for (int d = threadIdx.x * W; d < D; d += blockDim.x * W) {
    float y[W];
    load_vec<W>(yr + d, y);
#pragma unroll
    for (int e = 0; e < W; ++e) ss = fmaf(y[e], y[e], ss);
  }
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(D) + a.eps);
  for (int d = threadIdx.x * W; d < D; d += blockDim.x * W) {
    float y[W], x[W], w[W];
    load_vec<W>(yr + d, y);
    load_vec<W>(xr + d, x);
    load_vec<W>(a.w + d, w);
#pragma unroll
    for (int e = 0; e < W; ++e) x[e] += a.mult * (y[e] * inv) * w[e];
    store_vec(xr + d, x);
  }
  if (a.R > 0) {
    const int s = a.seq_of_row[t];
    const int pos = a.positions[t], slot = a.state_slots[s];
    if (slot >= 0 && pos >= a.context_lens[s] - a.R) {
      const float* src = a.unit + static_cast<long long>(t) * D;
      float* dst = a.ring + (static_cast<long long>(slot) * a.R + pos % a.R) * D;
      for (int d = threadIdx.x; d < D; d += blockDim.x) dst[d] = src[d];
    }
  }
}

template <typename T, int RB>
static int launch_finish(const FinishArgs& a, cudaStream_t s) {
  const size_t smem = (static_cast<size_t>(RB) * (a.D + a.side_dim) + 40) * sizeof(float);
  if (smem > 48 * 1024) cudaFuncSetAttribute(parallel_finish_kernel<T, RB>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
  TIE_LAUNCH((parallel_finish_kernel<T, RB>), ceil_div(a.T, RB), 256, smem, s, a);
  TIE_RETURN_LAUNCH("parallel_finish");
}

}  // namespace tie

using namespace tie;

TIE_API int tie_pair_hash_add(int dtype, float* x, const void* table, const int* tokens, const int* positions,
                              const int* seq_of_row, const int* query_start, const int* state_slots, int* prev_state,
                              int buckets, long long mul_prev, long long mul_cur, int rows, int dim, cudaStream_t s) {
  TIE_REQUIRE(rows >= 0 && dim > 0 && buckets > 0 && prev_state != nullptr, "pair_hash_add: bad sizes rows=%d dim=%d buckets=%d",
              rows, dim, buckets);
  if (rows == 0) return kOk;
  if (dtype == TIE_F32) {
    TIE_LAUNCH((pair_hash_add_kernel<float>), rows, 128, 0, s, x, static_cast<const float*>(table), tokens, positions, seq_of_row,
               query_start, state_slots, prev_state, buckets, mul_prev, mul_cur, dim);
  } else if (dtype == TIE_BF16) {
    TIE_LAUNCH((pair_hash_add_kernel<__nv_bfloat16>), rows, 128, 0, s, x, static_cast<const __nv_bfloat16*>(table), tokens,
               positions, seq_of_row, query_start, state_slots, prev_state, buckets, mul_prev, mul_cur, dim);
  } else {
    set_error("pair_hash_add: unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("pair_hash_add");
}

TIE_API int tie_add_row_vector(float* x, const float* vec, int rows, int dim, cudaStream_t s) {
  TIE_REQUIRE(rows >= 0 && dim > 0 && x != nullptr && vec != nullptr, "add_row_vector: bad arguments rows=%d dim=%d", rows, dim);
  const long long total = static_cast<long long>(rows) * dim;
  if (total == 0) return kOk;
  TIE_LAUNCH(add_row_vector_kernel, ceil_div(total, 256), 256, 0, s, x, vec, dim, total);
  TIE_RETURN_LAUNCH("add_row_vector");
}

TIE_API int tie_group_norm_taps(int dtype, float* x, const void* delta, const float* part, long long part_stride, int splits,
                                const int* rows, int n, int dim, int groups, float eps, const float* w_a, const float* w_b,
                                const float* taps_a, const float* taps_b, int taps, void* out_a, void* out_b, float* unit,
                                const float* ring, const int* seq_of_row, const int* positions, const int* query_start,
                                const int* context_lens, const int* state_slots, int tile_rows, cudaStream_t s) {
  TIE_REQUIRE(n >= 0 && dim > 0 && groups > 0 && dim % groups == 0, "group_norm_taps: %d columns do not split into %d equal groups",
              dim, groups);
  TIE_REQUIRE(taps >= 0 && taps <= kMaxTaps, "group_norm_taps: at most %d taps, got %d", kMaxTaps, taps);
  TIE_REQUIRE(w_a != nullptr && out_a != nullptr && (w_b == nullptr || out_b != nullptr), "group_norm_taps: an output without a buffer");
  TIE_REQUIRE(taps == 0 || (taps_a != nullptr && (w_b == nullptr || taps_b != nullptr) && seq_of_row != nullptr && positions != nullptr &&
                            query_start != nullptr && context_lens != nullptr && state_slots != nullptr &&
                            (taps == 1 || (unit != nullptr && ring != nullptr))),
              "group_norm_taps: taps need their weights, the step's index arrays and the state ring");
  TIE_REQUIRE(taps == 0 || (rows == nullptr && delta == nullptr && part == nullptr),
              "group_norm_taps: gathered rows and a delta go with taps = 0 only (the rows before a row are renormed from x)");
  TIE_REQUIRE(part == nullptr || (delta == nullptr && splits >= 1), "group_norm_taps: give a delta or partial sums, not both");
  if (n == 0) return kOk;
  NormTapsArgs a{};
  a.x = x;
  a.delta = Delta{delta, part, part_stride, splits};
  a.rows = rows;
  a.n = n, a.D = dim, a.groups = groups, a.eps = eps;
  a.w_a = w_a, a.w_b = w_b, a.taps_a = taps_a, a.taps_b = taps_b, a.taps = taps;
  a.out_a = out_a, a.out_b = out_b, a.unit = unit, a.ring = ring;
  a.seq_of_row = seq_of_row, a.positions = positions, a.query_start = query_start, a.context_lens = context_lens;
  a.state_slots = state_slots;
  if (taps > 0) {
    // rows a tile: as many (up to 8) as still leave every SM a block or two; measured at 2,048 rows of 2,048 columns with L2
    // flushed, tiles of 1, 2, 4, 8, 16 rows take 41, 33, 27, 23, 29 us; 4 columns a thread where the groups allow
    const int tile = tile_rows > 0 ? tile_rows : n >= 8 * 148 ? 8 : n >= 4 * 148 ? 4 : n >= 2 * 148 ? 2 : 1;
    TIE_REQUIRE(tile <= 64, "group_norm_taps: tiles of at most 64 rows, got %d", tile);
    const bool wide = dim % 4 == 0 && (dim / groups) % 4 == 0;
    const size_t tile_smem = (static_cast<size_t>(tile + taps - 1) * groups + 4 * tile) * sizeof(float);
    TIE_REQUIRE(tile_smem <= 48 * 1024, "group_norm_taps: %d groups are too many", groups);
#define TIE_TAPS_LAUNCH(TYPE, W, N) TIE_LAUNCH((group_norm_taps_tile_kernel<TYPE, W, N>), ceil_div(n, tile), 256, tile_smem, s, a, tile)
#define TIE_TAPS_CASE(TYPE, W)                \
  switch (taps) {                             \
    case 1: TIE_TAPS_LAUNCH(TYPE, W, 1); break; \
    case 2: TIE_TAPS_LAUNCH(TYPE, W, 2); break; \
    case 3: TIE_TAPS_LAUNCH(TYPE, W, 3); break; \
    case 4: TIE_TAPS_LAUNCH(TYPE, W, 4); break; \
    case 5: TIE_TAPS_LAUNCH(TYPE, W, 5); break; \
    case 6: TIE_TAPS_LAUNCH(TYPE, W, 6); break; \
    case 7: TIE_TAPS_LAUNCH(TYPE, W, 7); break; \
    default: TIE_TAPS_LAUNCH(TYPE, W, 8); break; \
  }
    if (dtype == TIE_F32) {
      if (wide) TIE_TAPS_CASE(float, 4)
      else TIE_TAPS_CASE(float, 1)
    } else if (dtype == TIE_BF16) {
      if (wide) TIE_TAPS_CASE(__nv_bfloat16, 4)
      else TIE_TAPS_CASE(__nv_bfloat16, 1)
    } else {
      set_error("group_norm_taps: unknown dtype code %d", dtype);
      return kBadArgument;
    }
#undef TIE_TAPS_LAUNCH
#undef TIE_TAPS_CASE
    TIE_RETURN_LAUNCH("group_norm_taps");
  }
  const bool summed = taps == 0 && (delta != nullptr || part != nullptr);
  const size_t smem = (static_cast<size_t>(groups) + (summed ? dim : 0)) * sizeof(float);
  TIE_REQUIRE(smem <= 200 * 1024, "group_norm_taps: a row of %d columns does not fit shared memory", dim);
  if (dtype == TIE_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(group_norm_taps_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    TIE_LAUNCH((group_norm_taps_kernel<float>), n, 256, smem, s, a);
  } else if (dtype == TIE_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(group_norm_taps_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    TIE_LAUNCH((group_norm_taps_kernel<__nv_bfloat16>), n, 256, smem, s, a);
  } else {
    set_error("group_norm_taps: unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("group_norm_taps");
}

TIE_API int tie_parallel_finish(int dtype, float* x, int rows, int dim, float mult, const void* delta_a, const float* part_a,
                                long long stride_a, int splits_a, const void* delta_b, const float* part_b, long long stride_b,
                                int splits_b, const int* tokens, const void* side_table, const void* side_gate,
                                const void* side_proj, const float* side_norm, int side_dim, float eps, const float* unit,
                                float* ring, int ring_rows, const int* seq_of_row, const int* positions,
                                const int* context_lens, const int* state_slots, cudaStream_t s) {
  TIE_REQUIRE(rows >= 0 && dim > 0 && side_dim >= 0 && ring_rows >= 0, "parallel_finish: bad sizes rows=%d dim=%d", rows, dim);
  TIE_REQUIRE((delta_a == nullptr || part_a == nullptr) && (delta_b == nullptr || part_b == nullptr),
              "parallel_finish: give a delta or partial sums, not both");
  TIE_REQUIRE(side_dim == 0 || (tokens != nullptr && side_table != nullptr && side_gate != nullptr && side_proj != nullptr &&
                                side_norm != nullptr), "parallel_finish: the token side input needs its tensors");
  TIE_REQUIRE(ring_rows == 0 || (unit != nullptr && ring != nullptr && seq_of_row != nullptr && positions != nullptr &&
                                 context_lens != nullptr && state_slots != nullptr), "parallel_finish: the ring needs the step's index arrays");
  if (rows == 0) return kOk;
  FinishArgs a{};
  a.x = x, a.T = rows, a.D = dim, a.mult = mult;
  a.a = Delta{delta_a, part_a, stride_a, splits_a};
  a.b = Delta{delta_b, part_b, stride_b, splits_b};
  a.tokens = tokens, a.side_table = side_table, a.side_gate = side_gate, a.side_proj = side_proj, a.side_norm = side_norm;
  a.side_dim = side_dim, a.eps = eps;
  a.unit = unit, a.ring = ring, a.R = ring_rows;
  a.seq_of_row = seq_of_row, a.positions = positions, a.context_lens = context_lens, a.state_slots = state_slots;
  const size_t one = (static_cast<size_t>(dim) + side_dim + 40) * sizeof(float);
  TIE_REQUIRE(one <= 200 * 1024, "parallel_finish: a row of %d columns does not fit shared memory", dim);
  // few rows with a side input: a cluster a row, while all clusters of the launch fit the GPU at once twice over
  const bool cluster = side_dim > 0 && rows * kFinishCluster <= 2 * 148 && one <= 100 * 1024;
  if (dtype == TIE_F32) return cluster ? launch_finish_cluster<float>(a, s) : launch_finish<float, 1>(a, s);
  if (dtype == TIE_BF16) return cluster ? launch_finish_cluster<__nv_bfloat16>(a, s) : launch_finish<__nv_bfloat16, 1>(a, s);
  set_error("parallel_finish: unknown dtype code %d", dtype);
  return kBadArgument;
}

// x += mult * (delta_a + delta_b) and copy = x in the storage type.
TIE_API int tie_parallel_sum(int dtype, float* x, void* copy, int rows, int dim, float mult, const void* delta_a, const float* part_a,
                             long long stride_a, int splits_a, const void* delta_b, const float* part_b, long long stride_b,
                             int splits_b, cudaStream_t s) {
  TIE_REQUIRE(rows >= 0 && dim > 0 && x != nullptr && copy != nullptr, "parallel_sum: bad arguments rows=%d dim=%d", rows, dim);
  TIE_REQUIRE((delta_a == nullptr || part_a == nullptr) && (delta_b == nullptr || part_b == nullptr),
              "parallel_sum: give a delta or partial sums, not both");
  if (rows == 0) return kOk;
  const Delta da{delta_a, part_a, stride_a, splits_a}, db{delta_b, part_b, stride_b, splits_b};
  const bool wide = dim % 4 == 0 && (part_a == nullptr || stride_a % 4 == 0) && (part_b == nullptr || stride_b % 4 == 0);
  if (dtype == TIE_F32) {
    if (wide) TIE_LAUNCH((parallel_sum_kernel<float, 4>), rows, 256, 0, s, x, static_cast<float*>(copy), dim, mult, da, db);
    else TIE_LAUNCH((parallel_sum_kernel<float, 1>), rows, 256, 0, s, x, static_cast<float*>(copy), dim, mult, da, db);
  } else if (dtype == TIE_BF16) {
    if (wide) TIE_LAUNCH((parallel_sum_kernel<__nv_bfloat16, 4>), rows, 256, 0, s, x, static_cast<__nv_bfloat16*>(copy), dim, mult, da, db);
    else TIE_LAUNCH((parallel_sum_kernel<__nv_bfloat16, 1>), rows, 256, 0, s, x, static_cast<__nv_bfloat16*>(copy), dim, mult, da, db);
  } else {
    set_error("parallel_sum: unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("parallel_sum");
}

// g[t, i] = gelu_tanh(pre[t, i]) * table[tokens[t], i]; pre float [rows, side_dim], g and table in the storage type.
TIE_API int tie_side_gate_act(int dtype, const float* pre, const void* table, const int* tokens, void* g, int rows, int side_dim,
                              cudaStream_t s) {
  TIE_REQUIRE(rows >= 0 && side_dim > 0 && pre != nullptr && table != nullptr && tokens != nullptr && g != nullptr,
              "side_gate_act: bad arguments rows=%d side_dim=%d", rows, side_dim);
  const long long total = static_cast<long long>(rows) * side_dim;
  if (total == 0) return kOk;
  if (dtype == TIE_F32) {
    TIE_LAUNCH((side_gate_act_kernel<float>), ceil_div(total, 256), 256, 0, s, pre, static_cast<const float*>(table), tokens,
               static_cast<float*>(g), side_dim, total);
  } else if (dtype == TIE_BF16) {
    TIE_LAUNCH((side_gate_act_kernel<__nv_bfloat16>), ceil_div(total, 256), 256, 0, s, pre, static_cast<const __nv_bfloat16*>(table),
               tokens, static_cast<__nv_bfloat16*>(g), side_dim, total);
  } else {
    set_error("side_gate_act: unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("side_gate_act");
}

// x += mult * y / rms(y) * w (all float), then the rows of `unit` that are a request's last ring_rows go to its ring.
TIE_API int tie_side_finish(float* x, const float* y, int rows, int dim, float mult, float eps, const float* w, const float* unit,
                            float* ring, int ring_rows, const int* seq_of_row, const int* positions, const int* context_lens,
                            const int* state_slots, cudaStream_t s) {
  TIE_REQUIRE(rows >= 0 && dim > 0 && x != nullptr && y != nullptr && w != nullptr && ring_rows >= 0, "side_finish: bad arguments rows=%d dim=%d", rows, dim);
  TIE_REQUIRE(ring_rows == 0 || (unit != nullptr && ring != nullptr && seq_of_row != nullptr && positions != nullptr &&
                                 context_lens != nullptr && state_slots != nullptr), "side_finish: the ring needs the step's index arrays");
  if (rows == 0) return kOk;
  SideFinishArgs a{x, y, dim, mult, eps, w, unit, ring, ring_rows, seq_of_row, positions, context_lens, state_slots};
  if (dim % 4 == 0) TIE_LAUNCH(side_finish_kernel<4>, rows, 256, 0, s, a);
  else TIE_LAUNCH(side_finish_kernel<1>, rows, 256, 0, s, a);
  TIE_RETURN_LAUNCH("side_finish");
}
