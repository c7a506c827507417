// Causal attention whose scores are mixed across heads before the softmax, with an optional sink in the softmax:
//
//   raw[g, j]  = q_g . k_(kv head of g), j                       every query head g of the row, float
//   s[h, j]    = scale * sum_g mix[h, g] * raw[g, j]             (mix null: s = scale * raw)
//   p[h, j]    = exp(s[h, j]) / (sink + sum_j' exp(s[h, j']))    sink = 1: one more key of score 0 that has no value
//   out[h]     = sum_j p[h, j] * v_(kv head of h), j
//
// Because a head's weights need every head's scores, one block owns ALL heads of a query row (or of one split of a
// single row's keys) and walks the keys in tiles: raw scores of the tile for all heads (a lane per key, the key read
// once per kv head), the mix and an online softmax per head (a warp per head), then the weighted values (a thread
// per output element). Keys of `dim`, values of `vdim`, any sizes, float or bfloat16 storage, float arithmetic.
//
//   rope_pairs_unit_append   between the stacked q/k/v product and attention, one block per token: the first `rot`
//                            dimensions of every q and k head are turned in neighbouring pairs (2i, 2i+1) by
//                            position * inv_freq[i]; then each head is divided by its root mean square (unit = 1);
//                            q back in place, k and v into the cache planes at the token's slot.
#include <math.h>

#include "common.cuh"
#include "launchers.h"

namespace tie {

struct PairPrepArgs {
  void* proj;
  long long stride;
  int q_off, k_off, v_off;
  const float* inv_freq;
  int rot;
  int unit;
  float eps;
  const int* positions;
  const int* slots;
  void* k_cache;
  void* v_cache;
  int q_heads, kv_heads, dim, vdim, page_size;
};

template <typename T>
__global__ void __launch_bounds__(256) rope_pairs_unit_append_kernel(PairPrepArgs a) {
  pdl_sync();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  const float pos = static_cast<float>(a.positions[t]);
  const int slot = a.slots[t];
  T* base = static_cast<T*>(a.proj) + static_cast<long long>(t) * a.stride;
  const int half = a.dim / 2;
  for (int head = warp; head < a.q_heads + a.kv_heads; head += nwarps) {
    const bool is_q = head < a.q_heads;
    const int c = is_q ? head : head - a.q_heads;
    T* src = base + (is_q ? a.q_off : a.k_off) + static_cast<long long>(c) * a.dim;
    T* dst = src;
    if (!is_q) {
      if (slot < 0) continue;
      const int page = slot / a.page_size, off = slot % a.page_size;
      dst = static_cast<T*>(a.k_cache) + ((static_cast<long long>(page) * a.kv_heads + c) * a.page_size + off) * a.dim;
    }
    // a lane keeps its pairs in registers over the two passes only when the head is small; otherwise it reads twice
    float ss = 0.0f;
    for (int i = lane; i < half; i += 32) {
      float u = ld(src + 2 * i), v = ld(src + 2 * i + 1);
      if (2 * i < a.rot) {
        float sn, cs;
        sincosf(pos * a.inv_freq[i], &sn, &cs);
        const float ru = u * cs - v * sn, rv = v * cs + u * sn;
        u = ru, v = rv;
      }
      ss = fmaf(u, u, fmaf(v, v, ss));
    }
    ss = warp_sum(ss);
    const float inv = a.unit ? 1.0f / sqrtf(ss / static_cast<float>(a.dim) + a.eps) : 1.0f;
    for (int i = lane; i < half; i += 32) {
      float u = ld(src + 2 * i), v = ld(src + 2 * i + 1);
      if (2 * i < a.rot) {
        float sn, cs;
        sincosf(pos * a.inv_freq[i], &sn, &cs);
        const float ru = u * cs - v * sn, rv = v * cs + u * sn;
        u = ru, v = rv;
      }
      st(dst + 2 * i, u * inv);
      st(dst + 2 * i + 1, v * inv);
    }
  }
  if (slot >= 0) {
    const int page = slot / a.page_size, off = slot % a.page_size;
    for (int e = threadIdx.x; e < a.kv_heads * a.vdim; e += blockDim.x) {
      const int c = e / a.vdim, d = e - c * a.vdim;
      static_cast<T*>(a.v_cache)[((static_cast<long long>(page) * a.kv_heads + c) * a.page_size + off) * a.vdim + d] =
          base[a.v_off + e];
    }
  }
}

struct MixedArgs {
  const void* q;
  long long q_stride;
  const void* k_cache;      // [pages, kv_heads, page_size, dim]
  const void* v_cache;      // [pages, kv_heads, page_size, vdim]
  void* out;                // [T, heads * vdim]
  const float* mix;         // [heads, heads] or null
  const int* seq_of_row;
  const int* query_start;
  const int* context_lens;
  const int* block_tables;
  int max_blocks;
  int rows;
  int heads, kv_heads, dim, vdim, page_size;
  float scale;
  int sink;
  // split mode (seq_list != null): one query row per listed sequence, keys cut into splits
  const int* seq_list;
  int n_list, split_keys, max_splits;
  float* scratch;           // [n_list, heads, max_splits, vdim + 2]
};

constexpr int kMixTile = 64;        // keys a tile
constexpr int kMixThreads = 256;
constexpr int kMixMaxPerThread = 32; // output elements a thread

template <typename T, int EPT>
__global__ void __launch_bounds__(kMixThreads) attention_mixed_kernel(MixedArgs a) {
  pdl_sync();
  extern __shared__ float smem[];
  const int H = a.heads, G = a.kv_heads, per = H / G;
  float* qs = smem;                           // [H * dim]
  float* raw = qs + H * a.dim;                // [H * tile]
  float* pw = raw + H * kMixTile;             // [H * tile]
  float* mixs = pw + H * kMixTile;            // [H * H]
  float* m_run = mixs + H * H;                // [H]
  float* l_run = m_run + H;
  float* corr = l_run + H;
  int* key_row = reinterpret_cast<int*>(corr + H);    // [tile]: row of the key in kv head 0's part of its page
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = kMixThreads / 32;
  const bool split_mode = a.seq_list != nullptr;
  int t, s, lo, hi, split = 0, li = 0;
  if (split_mode) {
    li = blockIdx.x, split = blockIdx.y;
    s = a.seq_list[li];
    t = a.query_start[s];
    const int pos = a.context_lens[s] - 1;
    lo = split * a.split_keys;
    if (lo > pos) return;
    hi = split == a.max_splits - 1 ? pos : min(pos, lo + a.split_keys - 1);
  } else {
    t = blockIdx.x;
    s = a.seq_of_row[t];
    const int q0 = a.query_start[s], q1 = a.query_start[s + 1];
    lo = 0;
    hi = a.context_lens[s] - (q1 - q0) + (t - q0);
  }
  const int* table = a.block_tables + static_cast<long long>(s) * a.max_blocks;
  const T* qv = static_cast<const T*>(a.q) + static_cast<long long>(t) * a.q_stride;
  for (int e = threadIdx.x; e < H * a.dim; e += kMixThreads) qs[e] = ld(qv + e);
  for (int e = threadIdx.x; e < H * H; e += kMixThreads) mixs[e] = a.mix != nullptr ? a.mix[e] : (e / H == e % H ? 1.0f : 0.0f);
  const bool with_sink = a.sink != 0 && split == 0;
  for (int h = threadIdx.x; h < H; h += kMixThreads) {
    m_run[h] = with_sink ? 0.0f : -INFINITY;
    l_run[h] = with_sink ? 1.0f : 0.0f;
  }
  float acc[EPT];
#pragma unroll
  for (int i = 0; i < EPT; ++i) acc[i] = 0.0f;
  const int out_elems = H * a.vdim;
  const T* kc = static_cast<const T*>(a.k_cache);
  const T* vc = static_cast<const T*>(a.v_cache);
  constexpr int V = Vec16<T>::N;
  const bool wide = a.dim % V == 0;
  __syncthreads();

  for (int base = lo; base <= hi; base += kMixTile) {
    const int count = min(kMixTile, hi - base + 1);
    for (int jj = threadIdx.x; jj < count; jj += kMixThreads) {
      const int j = base + jj;
      key_row[jj] = table[j / a.page_size] * G * a.page_size + j % a.page_size;
    }
    __syncthreads();
    // raw scores: an item is (kv head, 32 keys); a lane owns a key and up to four heads of the group at a time
    const int chunks = (count + 31) / 32;
    for (int item = warp; item < G * chunks; item += nwarps) {
      const int c = item / chunks, jj = (item - c * chunks) * 32 + lane;
      if (jj >= count) continue;
      const T* kr = kc + (static_cast<long long>(key_row[jj]) + c * a.page_size) * a.dim;
      for (int g0 = 0; g0 < per; g0 += 4) {
        float dot[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        const float* q0 = qs + (c * per + g0) * a.dim;
        const int gn = min(4, per - g0);
        if (wide) {
          for (int d = 0; d < a.dim; d += V) {
            Vec16<T> kv;
            kv.load(kr + d);
#pragma unroll
            for (int g = 0; g < 4; ++g)
              if (g < gn) {
#pragma unroll
                for (int e = 0; e < V; ++e) dot[g] = fmaf(q0[g * a.dim + d + e], kv.v[e], dot[g]);
              }
          }
        } else {
          for (int d = 0; d < a.dim; ++d) {
            const float kd = ld(kr + d);
#pragma unroll
            for (int g = 0; g < 4; ++g)
              if (g < gn) dot[g] = fmaf(q0[g * a.dim + d], kd, dot[g]);
          }
        }
#pragma unroll
        for (int g = 0; g < 4; ++g)
          if (g < gn) raw[(c * per + g0 + g) * kMixTile + jj] = dot[g];
      }
    }
    __syncthreads();
    // the mix and the online softmax: a warp per head
    for (int h = warp; h < H; h += nwarps) {
      float sc[kMixTile / 32];
      float tile_max = -INFINITY;
#pragma unroll
      for (int i = 0; i < kMixTile / 32; ++i) {
        const int jj = i * 32 + lane;
        float v = -INFINITY;
        if (jj < count) {
          float sum = 0.0f;
          for (int g = 0; g < H; ++g) sum = fmaf(mixs[h * H + g], raw[g * kMixTile + jj], sum);
          v = sum * a.scale;
        }
        sc[i] = v;
        tile_max = fmaxf(tile_max, v);
      }
      tile_max = warp_max(tile_max);
      const float m_old = m_run[h];
      const float m_new = fmaxf(m_old, tile_max);
      float sum = 0.0f;
#pragma unroll
      for (int i = 0; i < kMixTile / 32; ++i) {
        const int jj = i * 32 + lane;
        const float p = jj < count ? expf(sc[i] - m_new) : 0.0f;
        pw[h * kMixTile + jj] = p;
        sum += p;
      }
      sum = warp_sum(sum);
      if (lane == 0) {
        const float cr = m_old == -INFINITY ? 0.0f : expf(m_old - m_new);
        corr[h] = cr;
        m_run[h] = m_new;
        l_run[h] = l_run[h] * cr + sum;
      }
    }
    __syncthreads();
    // weighted values: a thread per output element
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
      const int e = threadIdx.x + i * kMixThreads;
      if (e < out_elems) {
        const int h = e / a.vdim, d = e - h * a.vdim;
        const long long col = static_cast<long long>(h / per) * a.page_size * a.vdim + d;
        const float* ph = pw + h * kMixTile;
        float v = acc[i] * corr[h];
        for (int jj = 0; jj < count; ++jj) v = fmaf(ph[jj], ld(vc + static_cast<long long>(key_row[jj]) * a.vdim + col), v);
        acc[i] = v;
      }
    }
    __syncthreads();
  }

  if (split_mode) {
    float* dst = a.scratch + (static_cast<long long>(li) * H * a.max_splits + split) * (a.vdim + 2);
    const long long head_stride = static_cast<long long>(a.max_splits) * (a.vdim + 2);
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
      const int e = threadIdx.x + i * kMixThreads;
      if (e < out_elems) {
        const int h = e / a.vdim, d = e - h * a.vdim;
        dst[h * head_stride + d] = acc[i];
      }
    }
    for (int h = threadIdx.x; h < H; h += kMixThreads) {
      dst[h * head_stride + a.vdim] = m_run[h];
      dst[h * head_stride + a.vdim + 1] = l_run[h];
    }
  } else {
    T* o = static_cast<T*>(a.out) + static_cast<long long>(t) * out_elems;
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
      const int e = threadIdx.x + i * kMixThreads;
      if (e < out_elems) {
        const float l = l_run[e / a.vdim];
        st(o + e, l > 0.0f ? acc[i] / l : 0.0f);
      }
    }
  }
}

template <typename T>
int launch_mixed(const MixedArgs& a, dim3 grid, cudaStream_t s) {
  const int H = a.heads;
  const size_t smem = (static_cast<size_t>(H) * a.dim + 2 * static_cast<size_t>(H) * kMixTile + static_cast<size_t>(H) * H + 3 * H) *
                          sizeof(float) + kMixTile * sizeof(int);
  if (smem > 200 * 1024) {
    set_error("attention_mixed: %d heads of %d need %zu bytes of shared memory", H, a.dim, smem);
    return kBadArgument;
  }
  const int per_thread = ceil_div(static_cast<long long>(H) * a.vdim, kMixThreads);
#define TIE_MIX_CASE(E)                                                                                            \
  do {                                                                                                             \
    if (smem > 48 * 1024)                                                                                          \
      cudaFuncSetAttribute(attention_mixed_kernel<T, E>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)); \
    TIE_LAUNCH((attention_mixed_kernel<T, E>), grid, kMixThreads, smem, s, a);                                     \
  } while (0)
  if (per_thread <= 1) TIE_MIX_CASE(1);
  else if (per_thread <= 2) TIE_MIX_CASE(2);
  else if (per_thread <= 4) TIE_MIX_CASE(4);
  else if (per_thread <= 8) TIE_MIX_CASE(8);
  else if (per_thread <= 16) TIE_MIX_CASE(16);
  else TIE_MIX_CASE(kMixMaxPerThread);
#undef TIE_MIX_CASE
  TIE_RETURN_LAUNCH("attention_mixed");
}

}  // namespace tie

using namespace tie;

TIE_API int tie_rope_pairs_unit_append(int dtype, void* proj, long long stride, int q_off, int k_off, int v_off,
                                       const float* inv_freq, int rot, int unit, float eps, const int* positions,
                                       const int* slots, void* k_cache, void* v_cache, int tokens, int q_heads, int kv_heads,
                                       int dim, int vdim, int page_size, cudaStream_t s) {
  TIE_REQUIRE(tokens >= 0 && q_heads > 0 && kv_heads > 0 && dim > 0 && vdim > 0 && page_size > 0, "rope_pairs_unit_append: bad sizes");
  TIE_REQUIRE(dim % 2 == 0 && rot % 2 == 0 && rot >= 0 && rot <= dim && (rot == 0 || inv_freq != nullptr),
              "rope_pairs_unit_append: heads of %d with %d rotated dimensions: both must be even, the second at most the first", dim, rot);
  if (tokens == 0) return kOk;
  PairPrepArgs a{proj, stride, q_off, k_off, v_off, inv_freq, rot, unit, eps, positions, slots, k_cache, v_cache,
                 q_heads, kv_heads, dim, vdim, page_size};
  if (dtype == TIE_F32) {
    TIE_LAUNCH((rope_pairs_unit_append_kernel<float>), tokens, 256, 0, s, a);
  } else if (dtype == TIE_BF16) {
    TIE_LAUNCH((rope_pairs_unit_append_kernel<__nv_bfloat16>), tokens, 256, 0, s, a);
  } else {
    set_error("rope_pairs_unit_append: unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("rope_pairs_unit_append");
}

// Rows [0, rows) of q against the keys up to each row's own position (seq_list null), or one row per listed sequence
// with its keys cut into splits of `split_keys` whose (sums, maximum, weight sum) go to scratch
// [n_list, heads, max_splits, vdim + 2] for tie_attention_merge.
TIE_API int tie_attention_mixed(int dtype, const void* q, long long q_stride, const void* k_cache, const void* v_cache, void* out,
                                const float* mix, const int* seq_of_row, const int* query_start, const int* context_lens,
                                const int* block_tables, int max_blocks, int rows, int heads, int kv_heads, int dim, int vdim,
                                int page_size, float scale, int sink, const int* seq_list, int n_list, int split_keys,
                                int max_splits, float* scratch, cudaStream_t s) {
  TIE_REQUIRE(heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && vdim > 0 && page_size > 0,
              "attention_mixed: bad geometry heads=%d kv_heads=%d dim=%d vdim=%d", heads, kv_heads, dim, vdim);
  TIE_REQUIRE(static_cast<long long>(heads) * vdim <= static_cast<long long>(kMixThreads) * kMixMaxPerThread,
              "attention_mixed: %d heads of %d values are more than %d outputs a row", heads, vdim, kMixThreads * kMixMaxPerThread);
  MixedArgs a{};
  a.q = q, a.q_stride = q_stride, a.k_cache = k_cache, a.v_cache = v_cache, a.out = out, a.mix = mix;
  a.seq_of_row = seq_of_row, a.query_start = query_start, a.context_lens = context_lens, a.block_tables = block_tables;
  a.max_blocks = max_blocks, a.rows = rows;
  a.heads = heads, a.kv_heads = kv_heads, a.dim = dim, a.vdim = vdim, a.page_size = page_size;
  a.scale = scale, a.sink = sink;
  dim3 grid;
  if (seq_list != nullptr) {
    TIE_REQUIRE(split_keys > 0 && max_splits > 0 && scratch != nullptr && n_list >= 0, "attention_mixed: bad split geometry");
    if (n_list == 0) return kOk;
    a.seq_list = seq_list, a.n_list = n_list, a.split_keys = split_keys, a.max_splits = max_splits, a.scratch = scratch;
    grid = dim3(n_list, max_splits);
  } else {
    TIE_REQUIRE(rows >= 0 && seq_of_row != nullptr, "attention_mixed: rows need seq_of_row");
    if (rows == 0) return kOk;
    grid = dim3(rows);
  }
  if (dtype == TIE_F32) return launch_mixed<float>(a, grid, s);
  if (dtype == TIE_BF16) return launch_mixed<__nv_bfloat16>(a, grid, s);
  set_error("attention_mixed: unknown dtype code %d", dtype);
  return kBadArgument;
}
