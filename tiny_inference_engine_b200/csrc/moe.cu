// A feed-forward made of many small experts of which each token uses a few.
//
//   moe_route   one warp per token: scores from all experts' logits (float; a softmax over the experts, or a sigmoid
//               each), choice scores = scores + an optional correction per expert, the best `keep` of `groups` equal
//               blocks of consecutive experts by their best member (or by the sum of their few best), then the `top`
//               best experts of those groups by choice score (ties go to the lower index); weights are the chosen
//               experts' scores, over their sum (+ 1e-20) or as they are.
//   moe_align   one block: counts the (token, choice) pairs of every expert, gives each expert a range of rows
//               that is a whole number of tiles of `block_m` rows, and lists the pairs in that order (-1 pads a
//               tile). Also says which expert each tile belongs to and how many tiles there are, all on the
//               device: nothing of a step's routing is read by the host, so a step can be a captured graph.
//   moe_gemv, moe_gemv_blocks   the same products for tiles of 4 pairs (decode: an expert has a row or two): the
//               expert's weight rows are streamed once, a warp per output column (row-major weights) or per four
//               columns (weights in k-blocks).
//   moe_gather, moe_combine   for prompts in bfloat16: rows copied into the listed order ahead of the grouped products
//               on the tensor cores (gemm_tc.cu, tiles of 128 rows), and the weighted results back to their tokens.
//   moe_gemm    grouped products on the CUDA cores, one block per (tile of rows, 64 output columns): rows are
//               gathered through the list, weights are the tile's expert's. `first` reads token rows and writes a
//               row per pair; `second` reads a row per pair and writes weight * result as the pair's choice-th
//               partial sum of the token, float [top, tokens, N]: whoever adds the feed-forward's output to the
//               residual stream adds those `top` terms in order, in float.
#include <math.h>

#include <type_traits>

#include "common.cuh"

namespace tie {

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) v = ov, i = oi;
  }
}

// smem per warp: experts floats (scores), experts floats (work), groups floats, groups ints.
// score_fn 0: s = softmax over all experts; 1: s = sigmoid of each logit. Experts are chosen by s + correction
// (correction null: by s); a group counts as the sum of its `group_top` largest choice scores (1: its best member);
// experts outside the kept groups cannot be chosen (their choice score counts as minus infinity: choice scores may be
// negative). The weights are the chosen experts' s, over their sum (+ 1e-20) when `renorm`, else as they are.
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, long long ld_logits, int tokens,
                                                        int experts, int top, int groups, int keep, int score_fn,
                                                        const float* __restrict__ correction, int group_top, int renorm,
                                                        float weight_scale, int* __restrict__ ids, float* __restrict__ weights) {
  pdl_sync();
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long t = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + warp;
  if (t >= tokens) return;
  float* score = smem + warp * (2 * experts + 2 * groups);
  float* work = score + experts;
  float* gbest = work + experts;
  int* gsel = reinterpret_cast<int*>(gbest + groups);
  const float* z = logits + t * ld_logits;
  if (score_fn == 0) {
    float m = -INFINITY;
    for (int e = lane; e < experts; e += 32) m = fmaxf(m, z[e]);
    m = warp_max(m);
    float sum = 0.0f;
    for (int e = lane; e < experts; e += 32) {
      const float p = expf(z[e] - m);
      score[e] = p;
      sum += p;
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < experts; e += 32) score[e] *= inv;
  } else {
    for (int e = lane; e < experts; e += 32) score[e] = 1.0f / (1.0f + expf(-z[e]));
  }
  for (int e = lane; e < experts; e += 32) work[e] = score[e] + (correction != nullptr ? correction[e] : 0.0f);
  __syncwarp();
  const int per = experts / groups;
  if (keep < groups) {
    for (int g = lane; g < groups; g += 32) {
      // the sum of the group's `group_top` largest choice scores: the members in the order (score down, index up), each pick
      // the first one after the pick before
      float total = 0.0f, prev_v = INFINITY;
      int prev_i = -1;
      for (int k = 0; k < min(group_top, per); ++k) {
        float b = -INFINITY;
        int bi = -1;
        for (int e = 0; e < per; ++e) {
          const float v = work[g * per + e];
          const bool after = v < prev_v || (v == prev_v && e > prev_i) || (k == 0);
          if (after && (bi < 0 || v > b)) b = v, bi = e;
        }
        if (bi < 0) break;                    // nothing comparable is left (NaN)
        total += b;
        prev_v = b, prev_i = bi;
      }
      gbest[g] = total;
      gsel[g] = 0;
    }
    __syncwarp();
    for (int k = 0; k < keep; ++k) {
      float bv = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < groups; g += 32)
        if (!gsel[g] && (bi == 0x7fffffff || gbest[g] > bv)) bv = gbest[g], bi = g;
      warp_argmax(bv, bi);
      if (bi >= groups) bi = k;            // nothing comparable (a row of NaN): any group
      __syncwarp();
      if (lane == 0) gsel[bi] = 1;
      __syncwarp();
    }
    for (int e = lane; e < experts; e += 32)
      if (!gsel[e / per]) work[e] = -INFINITY;
    __syncwarp();
  }
  float total = 0.0f;
  float mine_w = 0.0f;
  int mine_e = 0;
  for (int k = 0; k < top; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < experts; e += 32)
      if (work[e] > bv) bv = work[e], bi = e;
    warp_argmax(bv, bi);
    if (bi >= experts) bi = k % experts;
    const float s = score[bi];
    total += s;
    if (lane == (k & 31)) mine_w = s, mine_e = bi;     // top <= 32 is checked by the launcher
    __syncwarp();
    if (lane == 0) work[bi] = -INFINITY;
    __syncwarp();
  }
  if (lane < top) {
    ids[t * top + lane] = mine_e;
    weights[t * top + lane] = (renorm ? mine_w / (total + 1e-20f) : mine_w) * weight_scale;     // the scale is a constant of the layer
  }
}

// meta[0] = number of tiles. smem: 2 * experts ints.
__global__ void __launch_bounds__(1024) moe_align_kernel(const int* __restrict__ ids, int pairs, int experts, int block_m,
                                                         int* __restrict__ sorted, int* __restrict__ tile_expert,
                                                         int* __restrict__ meta) {
  pdl_sync();
  extern __shared__ int ismem[];
  int* count = ismem;
  int* cursor = ismem + experts;
  __shared__ int total_rows;
  for (int e = threadIdx.x; e < experts; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) atomicAdd(&count[ids[i]], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int row = 0;
    for (int e = 0; e < experts; ++e) {
      cursor[e] = row;
      const int tiles = (count[e] + block_m - 1) / block_m;
      for (int i = 0; i < tiles; ++i) tile_expert[row / block_m + i] = e;
      row += tiles * block_m;
    }
    total_rows = row;
    meta[0] = row / block_m;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < total_rows; i += blockDim.x) sorted[i] = -1;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) sorted[atomicAdd(&cursor[ids[i]], 1)] = i;
}

// out rows for a tile of BM gathered rows against the 64 weight rows [n0, n0 + 64) of the tile's expert.
// SECOND false: a row = token pair / top of `a`; out[pair] in TO. SECOND true: a row = pair of `a`; the result times
// weights[pair] goes to partial[(pair % top)][pair / top] (float).
template <typename TI, typename TO, int BM, bool SECOND>
__global__ void __launch_bounds__(256) moe_gemm_kernel(const TI* __restrict__ a, long long lda, const TI* __restrict__ w,
                                                       long long w_expert_stride, TO* __restrict__ out, long long ldo,
                                                       float* __restrict__ partial, long long part_stride,
                                                       const float* __restrict__ weights, const int* __restrict__ sorted,
                                                       const int* __restrict__ tile_expert, const int* __restrict__ meta,
                                                       int top, int N, int K) {
  pdl_sync();
  constexpr int BN = 64, BK = 16, RM = BM / 16;
  const int tile = blockIdx.y;
  if (tile >= meta[0]) return;
  __shared__ float as[BK][BM + 4];
  __shared__ float ws[BK][BN + 4];
  __shared__ int pair_of[BM];
  const int tid = threadIdx.x;
  if (tid < BM) pair_of[tid] = sorted[tile * BM + tid];
  __syncthreads();
  const TI* we = w + static_cast<long long>(tile_expert[tile]) * w_expert_stride;
  const int n0 = blockIdx.x * BN;
  const int tm = (tid / 16) * RM, tn = (tid % 16) * 4;
  // loads: the weight tile is 64 x 16 (four k a thread); the row tile BM x 16
  const int wr = tid / 4, wk = (tid % 4) * 4;
  constexpr int A_PER = BM * BK / 256;                 // 4 (BM 64) or 1 (BM 16)
  const int ar = BM == 64 ? tid / 4 : tid / 16, ak = BM == 64 ? (tid % 4) * 4 : tid % 16;
  const int pa = pair_of[ar];
  const TI* arow = pa < 0 ? nullptr : a + static_cast<long long>(SECOND ? pa : pa / top) * lda;
  float acc[RM][4] = {};
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int k = k0 + wk + j, n = n0 + wr;
      ws[wk + j][wr] = (n < N && k < K) ? ld(we + static_cast<long long>(n) * K + k) : 0.0f;
    }
#pragma unroll
    for (int j = 0; j < A_PER; ++j) {
      const int k = k0 + ak + j;
      as[ak + j][ar] = (arow != nullptr && k < K) ? ld(arow + k) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float av[RM], wv[4];
#pragma unroll
      for (int i = 0; i < RM; ++i) av[i] = as[k][tm + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) wv[j] = ws[k][tn + j];
#pragma unroll
      for (int i = 0; i < RM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < RM; ++i) {
    const int pair = pair_of[tm + i];
    if (pair < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tn + j;
      if (n >= N) continue;
      if (SECOND) partial[(pair % top) * part_stride + static_cast<long long>(pair / top) * N + n] = weights[pair] * acc[i][j];
      else st(out + static_cast<long long>(pair) * ldo + n, acc[i][j]);
    }
  }
}

// Few rows per expert (decode): tiles of 4 pairs, one warp per (tile, output column). The warp streams its weight row
// once with 16-byte loads and keeps one sum per pair; the pairs' input rows come from L1/L2. Needs K in whole vectors.
template <typename TI, typename TO, bool SECOND>
__global__ void __launch_bounds__(256) moe_gemv_kernel(const TI* __restrict__ a, long long lda, const TI* __restrict__ w,
                                                       long long w_expert_stride, TO* __restrict__ out, long long ldo,
                                                       float* __restrict__ partial, long long part_stride,
                                                       const float* __restrict__ weights, const int* __restrict__ sorted,
                                                       const int* __restrict__ tile_expert, const int* __restrict__ meta,
                                                       int top, int N, int K) {
  pdl_sync();
  constexpr int V = Vec16<TI>::N, MT = 4;
  const int tile = blockIdx.y;
  if (tile >= meta[0]) return;
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (n >= N) return;
  int pair[MT];
  const TI* arow[MT];
#pragma unroll
  for (int i = 0; i < MT; ++i) {
    pair[i] = sorted[tile * MT + i];
    arow[i] = pair[i] < 0 ? nullptr : a + static_cast<long long>(SECOND ? pair[i] : pair[i] / top) * lda;
  }
  const TI* wr = w + static_cast<long long>(tile_expert[tile]) * w_expert_stride + static_cast<long long>(n) * K;
  float acc[MT] = {};
  for (int k = lane * V; k < K; k += 32 * V) {
    Vec16<TI> wv;
    wv.load(wr + k);
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      if (arow[i] != nullptr) {
        Vec16<TI> av;
        av.load(arow[i] + k);
#pragma unroll
        for (int j = 0; j < V; ++j) acc[i] = fmaf(av.v[j], wv.v[j], acc[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MT; ++i) {
    const float v = warp_sum(acc[i]);
    if (lane == 0 && pair[i] >= 0) {
      if (SECOND) partial[(pair[i] % top) * part_stride + static_cast<long long>(pair[i] / top) * N + n] = weights[pair[i]] * v;
      else st(out + static_cast<long long>(pair[i]) * ldo + n, v);
    }
  }
}

// Many rows per expert (prompts): the pairs' input rows are copied into the listed order, so that the grouped product
// on the tensor cores reads a dense operand whose tiles of 128 rows belong to one expert each; rows that pad a tile
// are zeros. 16 bytes a thread.
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ h, long long ldh, const int* __restrict__ sorted,
                                  const int* __restrict__ meta, int block_m, int top, T* __restrict__ out, int width) {
  pdl_sync();
  constexpr int V = Vec16<T>::N;
  const int row = blockIdx.x;
  if (row >= meta[0] * block_m) return;
  const int pair = sorted[row];
  for (int c = threadIdx.x * V; c < width; c += blockDim.x * V) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (pair >= 0) v = *reinterpret_cast<const uint4*>(h + static_cast<long long>(pair / top) * ldh + c);
    *reinterpret_cast<uint4*>(out + static_cast<long long>(row) * width + c) = v;
  }
}

// partial[pair % top][pair / top][:] = weights[pair] * y[row of the pair], float: the listed rows back to their tokens.
template <typename T>
__global__ void moe_combine_kernel(const T* __restrict__ y, const int* __restrict__ sorted, const int* __restrict__ meta,
                                   int block_m, int top, const float* __restrict__ weights, float* __restrict__ partial,
                                   long long part_stride, int width) {
  pdl_sync();
  const int row = blockIdx.x;
  if (row >= meta[0] * block_m) return;
  const int pair = sorted[row];
  if (pair < 0) return;
  const float wgt = weights[pair];
  float* dst = partial + (pair % top) * part_stride + static_cast<long long>(pair / top) * width;
  const T* src = y + static_cast<long long>(row) * width;
  for (int c = threadIdx.x * 4; c < width; c += blockDim.x * 4) {
    float v[4];
    load4(src + c, v);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] *= wgt;
    store4(dst + c, v);
  }
}

// The same for bfloat16 weights stored in k-blocks, [ceil(K / 64)][w_rows][64] (this expert's rows at expert * N): a
// warp takes four neighbouring output columns, eight lanes a column, so that one load instruction of the warp is 512
// consecutive bytes of a k-block (four rows' 64 elements) and a block's eight warps read 4 KB in a row; a lane sums its
// eighth of every k-block, and the eight lanes of a column add up at the end.
template <bool SECOND>
__global__ void __launch_bounds__(256) moe_gemv_blocks_kernel(const __nv_bfloat16* __restrict__ a, long long lda,
                                                              const __nv_bfloat16* __restrict__ w, int w_rows,
                                                              __nv_bfloat16* __restrict__ out, long long ldo,
                                                              float* __restrict__ partial, long long part_stride,
                                                              const float* __restrict__ weights, const int* __restrict__ sorted,
                                                              const int* __restrict__ tile_expert, const int* __restrict__ meta,
                                                              int top, int N, int K) {
  pdl_sync();
  constexpr int MT = 4;
  const int tile = blockIdx.y;
  if (tile >= meta[0]) return;
  const int lane = threadIdx.x & 31, sub = lane >> 3, piece = lane & 7;
  const int n = (blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5)) * 4 + sub;
  const bool live = n < N;
  int pair[MT];
  const __nv_bfloat16* arow[MT];
#pragma unroll
  for (int i = 0; i < MT; ++i) {
    pair[i] = sorted[tile * MT + i];
    arow[i] = pair[i] < 0 ? nullptr : a + static_cast<long long>(SECOND ? pair[i] : pair[i] / top) * lda + piece * 8;
  }
  const __nv_bfloat16* wr = w + (static_cast<long long>(tile_expert[tile]) * N + (live ? n : 0)) * 64 + piece * 8;
  const long long kb_stride = static_cast<long long>(w_rows) * 64;
  float acc[MT] = {};
  const int k_blocks = (K + 63) >> 6;
#pragma unroll 4
  for (int kb = 0; kb < k_blocks; ++kb) {
    if (kb * 64 + piece * 8 >= K) break;                 // the last k-block may be short (K in whole vectors)
    Vec16<__nv_bfloat16> wv;
    wv.load(wr + kb * kb_stride);
#pragma unroll
    for (int i = 0; i < MT; ++i) {
      if (arow[i] != nullptr) {
        Vec16<__nv_bfloat16> av;
        av.load(arow[i] + kb * 64);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i] = fmaf(av.v[j], wv.v[j], acc[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MT; ++i) {
    float v = acc[i];
    v += __shfl_xor_sync(0xffffffffu, v, 1);
    v += __shfl_xor_sync(0xffffffffu, v, 2);
    v += __shfl_xor_sync(0xffffffffu, v, 4);
    if (piece == 0 && live && pair[i] >= 0) {
      if (SECOND) partial[(pair[i] % top) * part_stride + static_cast<long long>(pair[i] / top) * N + n] = weights[pair[i]] * v;
      else out[static_cast<long long>(pair[i]) * ldo + n] = __float2bfloat16_rn(v);
    }
  }
}

}  // namespace tie

using namespace tie;

// h [T, width] -> out [rows, width] in listed order (rows = meta[0] * block_m of at most max_rows). width in whole 16-byte vectors.
TIE_API int tie_moe_gather(int dtype, const void* h, long long ldh, const int* sorted, const int* meta, int block_m, int top,
                           void* out, int width, int max_rows, cudaStream_t s) {
  TIE_REQUIRE(dtype == TIE_BF16 && width % 8 == 0 && ldh % 8 == 0 && reinterpret_cast<uintptr_t>(h) % 16 == 0 &&
                  reinterpret_cast<uintptr_t>(out) % 16 == 0,
              "moe_gather: bfloat16 rows of %d in whole 16-byte vectors", width);
  if (max_rows <= 0) return kOk;
  TIE_LAUNCH((moe_gather_kernel<__nv_bfloat16>), max_rows, 128, 0, s, static_cast<const __nv_bfloat16*>(h), ldh, sorted, meta, block_m,
             top, static_cast<__nv_bfloat16*>(out), width);
  TIE_RETURN_LAUNCH("moe_gather");
}

TIE_API int tie_moe_combine(int dtype, const void* y, const int* sorted, const int* meta, int block_m, int top,
                            const float* weights, float* partial, long long part_stride, int width, int max_rows, cudaStream_t s) {
  TIE_REQUIRE(dtype == TIE_BF16 && width % 4 == 0, "moe_combine: bfloat16 rows of %d in whole 8-byte pieces", width);
  if (max_rows <= 0) return kOk;
  TIE_LAUNCH((moe_combine_kernel<__nv_bfloat16>), max_rows, 128, 0, s, static_cast<const __nv_bfloat16*>(y), sorted, meta, block_m,
             top, weights, partial, part_stride, width);
  TIE_RETURN_LAUNCH("moe_combine");
}

TIE_API int tie_moe_route(const float* logits, long long ld_logits, int tokens, int experts, int top, int groups, int keep,
                          int score_fn, const float* correction, int group_top, int renorm, float weight_scale, int* ids,
                          float* weights, cudaStream_t s) {
  TIE_REQUIRE((score_fn == 0 || score_fn == 1) && group_top >= 1, "moe_route: score function %d, %d members a group's score",
              score_fn, group_top);
  TIE_REQUIRE(experts > 0 && top > 0 && top <= 32 && top <= experts && groups > 0 && experts % groups == 0 && keep > 0 &&
                  keep <= groups && top <= keep * (experts / groups),
              "moe_route: bad routing experts=%d top=%d (at most 32) groups=%d keep=%d", experts, top, groups, keep);
  if (tokens <= 0) return kOk;
  const size_t smem = 4 * sizeof(float) * (2 * experts + 2 * groups);
  TIE_REQUIRE(smem <= 48 * 1024, "moe_route: %d experts exceed the kernel's shared memory", experts);
  TIE_LAUNCH(moe_route_kernel, ceil_div(tokens, 4), 128, smem, s, logits, ld_logits, tokens, experts, top, groups, keep, score_fn,
             correction, group_top, renorm, weight_scale, ids, weights);
  TIE_RETURN_LAUNCH("moe_route");
}

TIE_API int tie_moe_align(const int* ids, int pairs, int experts, int block_m, int* sorted, int* tile_expert, int* meta,
                          cudaStream_t s) {
  TIE_REQUIRE(experts > 0 && experts <= 4096 && (block_m == 4 || block_m == 16 || block_m == 64 || block_m == 128),
              "moe_align: bad sizes experts=%d block_m=%d", experts, block_m);
  if (pairs <= 0) return kOk;
  TIE_LAUNCH(moe_align_kernel, 1, 1024, 2 * experts * sizeof(int), s, ids, pairs, experts, block_m, sorted, tile_expert, meta);
  TIE_RETURN_LAUNCH("moe_align");
}

// The most tiles `pairs` pairs over `experts` experts can need.
TIE_API int tie_moe_max_tiles(int pairs, int experts, int block_m) {
  const int full = pairs / block_m;
  return full + (experts < pairs ? experts : pairs);
}

template <typename TI, typename TO>
static int launch_moe_gemm(int second, int block_m, const void* a, long long lda, const void* w, long long w_expert_stride,
                           void* out, long long ldo, float* partial, long long part_stride, const float* weights,
                           const int* sorted, const int* tile_expert, const int* meta, int max_tiles, int top, int N, int K,
                           int w_rows, cudaStream_t s) {
  if (block_m == 4 && w_rows > 0) {
    if constexpr (std::is_same<TI, __nv_bfloat16>::value) {
      const dim3 grid(ceil_div(N, 32), max_tiles);
      const __nv_bfloat16* ap = static_cast<const __nv_bfloat16*>(a);
      const __nv_bfloat16* wp = static_cast<const __nv_bfloat16*>(w);
      if (second) {
        TIE_LAUNCH((moe_gemv_blocks_kernel<true>), grid, 256, 0, s, ap, lda, wp, w_rows, static_cast<__nv_bfloat16*>(out), ldo, partial,
                   part_stride, weights, sorted, tile_expert, meta, top, N, K);
      } else {
        TIE_LAUNCH((moe_gemv_blocks_kernel<false>), grid, 256, 0, s, ap, lda, wp, w_rows, static_cast<__nv_bfloat16*>(out), ldo, partial,
                   part_stride, weights, sorted, tile_expert, meta, top, N, K);
      }
      TIE_RETURN_LAUNCH("moe_gemv_blocks");
    } else {
      set_error("moe_gemm: weights in k-blocks are bfloat16");
      return kBadArgument;
    }
  }
  if (block_m == 4) {
    const dim3 grid(ceil_div(N, 8), max_tiles);
    if (second) {
      TIE_LAUNCH((moe_gemv_kernel<TI, TO, true>), grid, 256, 0, s, static_cast<const TI*>(a), lda, static_cast<const TI*>(w),
                 w_expert_stride, static_cast<TO*>(out), ldo, partial, part_stride, weights, sorted, tile_expert, meta, top, N, K);
    } else {
      TIE_LAUNCH((moe_gemv_kernel<TI, TO, false>), grid, 256, 0, s, static_cast<const TI*>(a), lda, static_cast<const TI*>(w),
                 w_expert_stride, static_cast<TO*>(out), ldo, partial, part_stride, weights, sorted, tile_expert, meta, top, N, K);
    }
    TIE_RETURN_LAUNCH("moe_gemv");
  }
  const dim3 grid(ceil_div(N, 64), max_tiles);
#define TIE_MOE_CASE(BM, SECOND)                                                                                            \
  TIE_LAUNCH((moe_gemm_kernel<TI, TO, BM, SECOND>), grid, 256, 0, s, static_cast<const TI*>(a), lda, static_cast<const TI*>(w), \
             w_expert_stride, static_cast<TO*>(out), ldo, partial, part_stride, weights, sorted, tile_expert, meta, top, N, K)
  if (block_m == 64) {
    if (second) TIE_MOE_CASE(64, true);
    else TIE_MOE_CASE(64, false);
  } else {
    if (second) TIE_MOE_CASE(16, true);
    else TIE_MOE_CASE(16, false);
  }
#undef TIE_MOE_CASE
  TIE_RETURN_LAUNCH("moe_gemm");
}

// second 0: out[pair, :N] = w[expert] a[pair / top]; second 1: partial[pair % top][pair / top][:N] = weights[pair] * (w[expert] a[pair]).
// w is [experts, N, K] (an expert's rows K apart, experts w_expert_stride apart), or with w_rows > 0 (tiles of 4 rows only)
// the same rows one expert after the other stored in k-blocks, [ceil(K / 64)][w_rows][64].
TIE_API int tie_moe_gemm(int dtype, int second, int block_m, const void* a, long long lda, const void* w,
                         long long w_expert_stride, void* out, long long ldo, float* partial, long long part_stride,
                         const float* weights, const int* sorted, const int* tile_expert, const int* meta, int max_tiles,
                         int top, int N, int K, int w_rows, cudaStream_t s) {
  TIE_REQUIRE(w_rows == 0 || (block_m == 4 && w_rows % N == 0), "moe_gemm: weights in k-blocks are read by the tiles of 4 rows only");
  TIE_REQUIRE(N > 0 && K > 0 && top > 0 && (block_m == 4 || block_m == 16 || block_m == 64) && max_tiles >= 0 && max_tiles <= 65535,
              "moe_gemm: bad sizes N=%d K=%d top=%d block_m=%d tiles=%d", N, K, top, block_m, max_tiles);
  if (max_tiles == 0) return kOk;
  if (block_m == 4) {
    const int v = dtype == TIE_BF16 ? 8 : 4;
    TIE_REQUIRE(K % v == 0 && lda % v == 0 && w_expert_stride % v == 0 && reinterpret_cast<uintptr_t>(a) % 16 == 0 &&
                    reinterpret_cast<uintptr_t>(w) % 16 == 0,
                "moe_gemm: tiles of 4 rows need K=%d and the row strides in whole 16-byte vectors", K);
  }
  if (dtype == TIE_F32)
    return launch_moe_gemm<float, float>(second, block_m, a, lda, w, w_expert_stride, out, ldo, partial, part_stride, weights, sorted,
                                         tile_expert, meta, max_tiles, top, N, K, w_rows, s);
  if (dtype == TIE_BF16)
    return launch_moe_gemm<__nv_bfloat16, __nv_bfloat16>(second, block_m, a, lda, w, w_expert_stride, out, ldo, partial, part_stride,
                                                         weights, sorted, tile_expert, meta, max_tiles, top, N, K, w_rows, s);
  set_error("unknown dtype code %d", dtype);
  return kBadArgument;
}
