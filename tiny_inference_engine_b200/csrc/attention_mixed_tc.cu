// Prompt portions of the attention whose scores are mixed across heads (attention_mixed.cu states what is computed), on the
// tensor cores: bfloat16 queries, keys and values, float accumulation, mma.sync m16n8k16.
//
// A head's weights need every head's scores, so one CTA owns ALL heads of a block of query positions. A warp is one
// (head, 16 query positions): per tile of 64 keys it forms its head's raw scores Q K^T and leaves them in shared memory;
// after a barrier it reads every head's raw scores at its own fragment coordinates, forms
// s'[h] = sum_g mix[h, g] raw[g] (the mix already times scale * log2 e), masks, updates its online softmax (which starts
// from the sink: maximum 0, sum 1) and adds P V, the float weights entering as two bfloat16 terms. The K and V tiles of
// every kv head of the sequence sit in shared memory once for all heads (cp.async, swizzled for ldmatrix), in one or
// two stages as shared memory allows.
//
// grid = (blocks of 16 * MT query positions, sequences that bring several tokens); block = 32 * heads * MT threads.
#include "attention_mma.cuh"

namespace tie {

struct MixedTcArgs {
  const __nv_bfloat16* q;
  long long q_stride;
  const __nv_bfloat16* k_cache;     // [pages, kv_heads, page_size, DK]
  const __nv_bfloat16* v_cache;     // [pages, kv_heads, page_size, DV]
  __nv_bfloat16* out;               // [T, heads * DV]
  const float* mix;                 // [heads, heads] or null
  const int* query_start;
  const int* context_lens;
  const int* block_tables;
  int max_blocks, heads, kv_heads, page_size, mt;
  float scale_log2;                 // scale * log2(e)
  int sink;
};

constexpr int kRawStride = kKeysPerTile + 8;      // floats a row of raw scores takes in shared memory

template <int DH>
__device__ __forceinline__ void load_tile_any(uint32_t dst, const __nv_bfloat16* __restrict__ plane, const int* __restrict__ table,
                                              int kvh, int kv_heads, int page_size, int key0, int hi) {
  constexpr int CPR = DH / 8;
  for (int id = threadIdx.x; id < kKeysPerTile * CPR; id += blockDim.x) {
    const int r = id / CPR, c = id - r * CPR;
    const int key = key0 + r;
    const bool valid = key <= hi;
    long long off = 0;
    if (valid) {
      const int page = table[key / page_size];
      off = (static_cast<long long>(page * kv_heads + kvh) * page_size + key % page_size) * DH + c * 8;
    }
    cp_async16(dst + swz<DH>(r, c), plane + off, valid ? 16 : 0);
  }
}

template <int DK, int DV, int STAGES, int MAXT>
__global__ void __launch_bounds__(MAXT) attn_mixed_prompt_tc_kernel(MixedTcArgs a) {
  pdl_sync();
  extern __shared__ __align__(128) uint8_t smem[];
  const int H = a.heads, G = a.kv_heads, per = H / G, MT = a.mt;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = warp % H, mt = warp / H;
  const int seq = blockIdx.y;
  const int t0 = a.query_start[seq];
  const int nq = a.query_start[seq + 1] - t0;
  const int q0 = blockIdx.x * 16 * MT;
  if (q0 >= nq) return;
  const int pos0 = a.context_lens[seq] - nq;
  const int hi_cta = pos0 + min(nq, q0 + 16 * MT) - 1;
  const int* table = a.block_tables + static_cast<long long>(seq) * a.max_blocks;

  constexpr int K_TILE = kKeysPerTile * DK * 2, V_TILE = kKeysPerTile * DV * 2;
  const int stage_bytes = G * (K_TILE + V_TILE);
  const uint32_t q_tile = smem_addr(smem);                                   // [H * MT * 16][DK]
  const uint32_t kv_base = q_tile + H * MT * 16 * DK * 2;
  float* raw = reinterpret_cast<float*>(smem + H * MT * 16 * DK * 2 + STAGES * stage_bytes);   // [H][MT * 16][kRawStride]
  float* mixs = raw + H * MT * 16 * kRawStride;                              // [H][H], times scale * log2 e

  // Q of this block's positions, every head: row (mt * H + h) * 16 + i of the tile
  constexpr int CPR = DK / 8;
  for (int id = threadIdx.x; id < H * MT * 16 * CPR; id += blockDim.x) {
    const int r = id / CPR, c = id - r * CPR;
    const int w = r >> 4, hh = w % H, qi = q0 + (w / H) * 16 + (r & 15);
    const bool valid = qi < nq;
    const __nv_bfloat16* src = a.q;
    if (valid) src = a.q + static_cast<long long>(t0 + qi) * a.q_stride + hh * DK + c * 8;
    cp_async16(q_tile + swz<DK>(r, c), src, valid ? 16 : 0);
  }
  cp_async_commit();
  for (int e = threadIdx.x; e < H * H; e += blockDim.x)
    mixs[e] = (a.mix != nullptr ? a.mix[e] : (e / H == e % H ? 1.0f : 0.0f)) * a.scale_log2;

  const int n_tiles = hi_cta / kKeysPerTile + 1;
  auto load_stage = [&](int tile) {
    const uint32_t dst = kv_base + (tile % STAGES) * stage_bytes;
    for (int c = 0; c < G; ++c) {
      load_tile_any<DK>(dst + c * K_TILE, a.k_cache, table, c, G, a.page_size, tile * kKeysPerTile, hi_cta);
      load_tile_any<DV>(dst + G * K_TILE + c * V_TILE, a.v_cache, table, c, G, a.page_size, tile * kKeysPerTile, hi_cta);
    }
  };
  if (STAGES == 2) {
    load_stage(0);
    cp_async_commit();
    cp_async_wait<1>();          // Q has landed
  } else {
    cp_async_wait<0>();
  }
  __syncthreads();
  uint32_t qf[DK / 16][4];
#pragma unroll
  for (int ks = 0; ks < DK / 16; ++ks) ldmatrix_x4(qf[ks], q_tile + swz<DK>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));

  const int gq = lane >> 2, tq = lane & 3;
  int row_pos[2];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int qi = q0 + mt * 16 + gq + 8 * half;
    row_pos[half] = qi < nq ? pos0 + qi : -1;
  }
  const int warp_hi = q0 + mt * 16 < nq ? pos0 + min(nq - 1, q0 + mt * 16 + 15) : -1;
  float m[2], l[2];
  m[0] = m[1] = a.sink ? 0.0f : -INFINITY;
  l[0] = l[1] = a.sink ? 1.0f : 0.0f;
  float acc[DV / 8][4];
#pragma unroll
  for (int j = 0; j < DV / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
  float* my_raw = raw + (static_cast<long long>(h) * MT + mt) * 16 * kRawStride;
  const float* mix_row = mixs + h * H;

  for (int i = 0; i < n_tiles; ++i) {
    if (STAGES == 2) {
      if (i + 1 < n_tiles) load_stage(i + 1);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      load_stage(i);
      cp_async_commit();
      cp_async_wait<0>();
    }
    __syncthreads();
    const int key0 = i * kKeysPerTile;
    const bool active = key0 <= warp_hi;          // the same for every head of this warp's positions
    const uint32_t stage = kv_base + (i % STAGES) * stage_bytes;
    float s[8][4];
    if (active) {
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
      qk_tile<DK, 8>(s, qf, stage + (h / per) * K_TILE, 0);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        *reinterpret_cast<float2*>(my_raw + gq * kRawStride + j * 8 + tq * 2) = make_float2(s[j][0], s[j][1]);
        *reinterpret_cast<float2*>(my_raw + (gq + 8) * kRawStride + j * 8 + tq * 2) = make_float2(s[j][2], s[j][3]);
      }
    }
    __syncthreads();
    if (active) {
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
      for (int g = 0; g < H; ++g) {
        const float w = mix_row[g];
        const float* src = raw + (static_cast<long long>(g) * MT + mt) * 16 * kRawStride;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float2 lo = *reinterpret_cast<const float2*>(src + gq * kRawStride + j * 8 + tq * 2);
          const float2 hi = *reinterpret_cast<const float2*>(src + (gq + 8) * kRawStride + j * 8 + tq * 2);
          s[j][0] = fmaf(w, lo.x, s[j][0]);
          s[j][1] = fmaf(w, lo.y, s[j][1]);
          s[j][2] = fmaf(w, hi.x, s[j][2]);
          s[j][3] = fmaf(w, hi.y, s[j][3]);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key0 + j * 8 + tq * 2 + (e & 1);
          if (key > row_pos[e >> 1]) s[j][e] = -INFINITY;
        }
      }
      softmax_update<DV, 8>(s, m, l, acc);
      pv_tile<DV, 8>(acc, s, stage + G * K_TILE + (h / per) * V_TILE, 0, true);
    }
    __syncthreads();
  }
  cp_async_wait<0>();

#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int qi = q0 + mt * 16 + gq + 8 * half;
    if (qi >= nq) continue;
    const float inv = l[half] > 0.0f ? 1.0f / l[half] : 0.0f;
    __nv_bfloat16* o = a.out + (static_cast<long long>(t0 + qi) * H + h) * DV;
#pragma unroll
    for (int j = 0; j < DV / 8; ++j)
      *reinterpret_cast<uint32_t*>(o + j * 8 + tq * 2) = pack_bf16(acc[j][2 * half] * inv, acc[j][2 * half + 1] * inv);
  }
}

// Shared memory of a block: Q tile, `stages` stages of every kv head's K and V tiles, raw scores, the mix.
static size_t mixed_tc_smem(int heads, int kv_heads, int dim, int vdim, int mt, int stages) {
  return static_cast<size_t>(heads) * mt * 16 * dim * 2 + static_cast<size_t>(stages) * kv_heads * kKeysPerTile * (dim + vdim) * 2 +
         static_cast<size_t>(heads) * mt * 16 * kRawStride * 4 + static_cast<size_t>(heads) * heads * 4;
}

constexpr size_t kMixedTcSmemLimit = 220 * 1024;

// (mt, stages) for a geometry, or mt = 0 when the kernel does not take it. Two blocks of 16 positions while the block stays at
// 256 threads; two stages where two blocks still fit an SM, else one stage if that lets two fit, else whatever fits alone.
static void mixed_tc_plan(int heads, int kv_heads, int dim, int vdim, int* mt, int* stages) {
  *mt = 0, *stages = 0;
  if (!((dim == 64 || dim == 128) && (vdim == 64 || vdim == 128)) || heads > 16 || heads % kv_heads != 0) return;
  const size_t pair = 110 * 1024;
  for (int m = heads <= 4 ? 2 : 1; m >= 1; --m) {
    const size_t two = mixed_tc_smem(heads, kv_heads, dim, vdim, m, 2), one = mixed_tc_smem(heads, kv_heads, dim, vdim, m, 1);
    const int st = two <= pair ? 2 : one <= pair ? 1 : two <= kMixedTcSmemLimit ? 2 : one <= kMixedTcSmemLimit ? 1 : 0;
    if (st > 0) {
      *mt = m, *stages = st;
      return;
    }
  }
}

template <int DK, int DV>
static int launch_mixed_tc(const MixedTcArgs& a, dim3 grid, int stages, size_t smem, cudaStream_t s) {
  const int threads = 32 * a.heads * a.mt;
#define TIE_MIXED_TC_CASE(ST, MAXT)                                                                                  \
  do {                                                                                                               \
    cudaFuncSetAttribute(attn_mixed_prompt_tc_kernel<DK, DV, ST, MAXT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                         static_cast<int>(smem));                                                                    \
    TIE_LAUNCH((attn_mixed_prompt_tc_kernel<DK, DV, ST, MAXT>), grid, threads, smem, s, a);                          \
  } while (0)
  if (threads <= 256) {
    if (stages == 2) TIE_MIXED_TC_CASE(2, 256);
    else TIE_MIXED_TC_CASE(1, 256);
  } else {
    if (stages == 2) TIE_MIXED_TC_CASE(2, 512);
    else TIE_MIXED_TC_CASE(1, 512);
  }
#undef TIE_MIXED_TC_CASE
  TIE_RETURN_LAUNCH("attention_mixed_tc");
}

}  // namespace tie

using namespace tie;

// 1 when tie_attention_mixed_tc takes this geometry (bfloat16 only), else 0.
TIE_API int tie_attention_mixed_tc_takes(int heads, int kv_heads, int dim, int vdim) {
  int mt, stages;
  mixed_tc_plan(heads, kv_heads, dim, vdim, &mt, &stages);
  return mt > 0 ? 1 : 0;
}

// Sequences 0 .. n_seqs-1 of the step each bring several tokens, at most max_queries.
TIE_API int tie_attention_mixed_tc(const void* q, long long q_stride, const void* k_cache, const void* v_cache, void* out,
                                   const float* mix, const int* query_start, const int* context_lens, const int* block_tables,
                                   int max_blocks, int n_seqs, int max_queries, int heads, int kv_heads, int dim, int vdim,
                                   int page_size, float scale, int sink, cudaStream_t s) {
  TIE_REQUIRE(heads > 0 && kv_heads > 0 && page_size > 0 && n_seqs >= 0 && max_queries >= 0, "attention_mixed_tc: bad sizes");
  int mt, stages;
  mixed_tc_plan(heads, kv_heads, dim, vdim, &mt, &stages);
  TIE_REQUIRE(mt > 0, "attention_mixed_tc: heads=%d kv_heads=%d dim=%d vdim=%d is served by the CUDA-core kernel", heads, kv_heads,
              dim, vdim);
  TIE_REQUIRE(q_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0, "attention_mixed_tc: q rows must start on 16 bytes");
  if (n_seqs == 0 || max_queries == 0) return kOk;
  MixedTcArgs a{};
  a.q = static_cast<const __nv_bfloat16*>(q), a.q_stride = q_stride;
  a.k_cache = static_cast<const __nv_bfloat16*>(k_cache), a.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  a.out = static_cast<__nv_bfloat16*>(out), a.mix = mix;
  a.query_start = query_start, a.context_lens = context_lens, a.block_tables = block_tables;
  a.max_blocks = max_blocks, a.heads = heads, a.kv_heads = kv_heads, a.page_size = page_size, a.mt = mt;
  a.scale_log2 = scale * 1.4426950408889634f, a.sink = sink;
  const dim3 grid(ceil_div(max_queries, 16 * mt), n_seqs);
  const size_t smem = mixed_tc_smem(heads, kv_heads, dim, vdim, mt, stages);
  if (dim == 64 && vdim == 64) return launch_mixed_tc<64, 64>(a, grid, stages, smem, s);
  if (dim == 64 && vdim == 128) return launch_mixed_tc<64, 128>(a, grid, stages, smem, s);
  if (dim == 128 && vdim == 64) return launch_mixed_tc<128, 64>(a, grid, stages, smem, s);
  return launch_mixed_tc<128, 128>(a, grid, stages, smem, s);
}
