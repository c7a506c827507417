// The attention whose scores are mixed across heads (attention_mixed.cu states what is computed), on the tensor cores:
// bfloat16 queries, keys and values, float accumulation, mma.sync m16n8k16. It serves portions of prompts (every query
// position against the keys up to its own) and single rows whose keys are cut into splits that attention_merge joins.
//
// A head's weights need every head's scores, so one CTA owns ALL heads of a block of query positions. A warp owns 16
// rows = (hpw query heads of one kv head) x (qpw query positions), hpw = gcd(heads / kv_heads, 16), qpw = 16 / hpw, so
// that also many heads fit a block of 16 warps: per tile of keys the warp forms its rows' raw scores Q K^T and leaves
// them in shared memory; after a barrier it reads every head's raw scores at its own fragment coordinates, forms
// s'[h] = sum_g mix[h, g] raw[g] (the mix already times scale * log2 e), masks, updates its online softmax (which starts
// from the sink: maximum 0, sum 1) and adds P V, the float weights entering as two bfloat16 terms.
//
// The K tile and the V tile of EVERY kv head sit in shared memory once for all heads (cp.async, swizzled for ldmatrix),
// one buffer each, loaded askew: the next K tile arrives while the mix, the softmax and P V of this one run, the next
// V tile while the next Q K^T runs. The tile has 64, 32 or 16 keys, as many as shared memory allows for the geometry.
// The Q tile is read into registers once and its room is then the V buffer's.
//
// grid = (blocks of nsub * qpw query positions, sequences) for prompts, (listed sequences, splits) for single rows;
// block = 32 * (heads / hpw) * nsub threads, at most 512.
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
  int max_blocks, heads, kv_heads, page_size;
  int hpw, qpw, nsub;               // heads and query positions of a warp's 16 rows; groups of qpw positions a block
  float scale_log2;                 // scale * log2(e)
  int sink;
  // single rows (seq_list != null): one query row per listed sequence, its keys cut into splits
  const int* seq_list;
  int split_keys, max_splits;
  float* scratch;                   // [n_list, heads, max_splits, DV + 2]
};

// Row offsets of a tile's keys in kv head 0's part of their pages (-1: outside [.., hi]), for the copies of both planes.
template <int KT>
__device__ __forceinline__ void tile_rows(int* rows, const int* __restrict__ table, int kv_heads, int page_size, int key0, int hi) {
  for (int r = threadIdx.x; r < KT; r += blockDim.x) {        // a block may have fewer threads than the tile has keys
    const int key = key0 + r;
    rows[r] = key <= hi ? table[key / page_size] * kv_heads * page_size + key % page_size : -1;
  }
}

// Copies the tile's rows of every kv head from one plane: tile c of KT rows at dst + c * KT * DH * 2.
template <int DH, int KT>
__device__ __forceinline__ void load_plane_tiles(uint32_t dst, const __nv_bfloat16* __restrict__ plane, const int* rows, int kv_heads,
                                                 int page_size) {
  constexpr int CPR = DH / 8;
  const int total = kv_heads * KT * CPR;
  for (int id = threadIdx.x; id < total; id += blockDim.x) {
    const int c = id % CPR, r = (id / CPR) % KT, kvh = id / (CPR * KT);
    const int row = rows[r];
    const bool valid = row >= 0;
    const long long off = valid ? (static_cast<long long>(row) + static_cast<long long>(kvh) * page_size) * DH + c * 8 : 0;
    cp_async16(dst + kvh * (KT * DH * 2) + swz<DH>(r, c), plane + off, valid ? 16 : 0);
  }
}

__device__ __forceinline__ void sts_f2(uint32_t addr, float x, float y) {
  asm volatile("st.shared.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(x), "f"(y) : "memory");
}
__device__ __forceinline__ float2 lds_f2(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ float lds_f(uint32_t addr) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1];" : "=f"(v) : "r"(addr));
  return v;
}

__device__ __forceinline__ void sts_u4(uint32_t addr, const uint32_t (&v)[4]) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]) : "memory");
}
__device__ __forceinline__ void lds_u4(uint32_t (&v)[4], uint32_t addr) {
  asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]) : "r"(addr));
}

// Q K^T of a warp's 16 rows against a K tile, like qk_tile, with the Q fragments of the first KREG k-steps in registers
// and the others in shared memory as the lanes left them (16 bytes a lane and k-step at `kept`).
template <int DK, int NT, int KREG>
__device__ __forceinline__ void qk_rows(float (&s)[NT][4], const uint32_t (&qf)[KREG][4], uint32_t kept, uint32_t k_tile) {
  const int lane = threadIdx.x & 31;
#pragma unroll
  for (int ks = 0; ks < DK / 16; ++ks) {
    uint32_t a[4];
    if (ks < KREG) {
#pragma unroll
      for (int e = 0; e < 4; ++e) a[e] = qf[ks < KREG ? ks : 0][e];
    } else {
      lds_u4(a, kept + (ks - KREG) * 512);
    }
#pragma unroll
    for (int np = 0; np < NT / 2; ++np) {
      uint32_t b[4];
      const int r = np * 16 + (lane & 7) + ((lane >> 4) << 3);
      const int c = ks * 2 + ((lane >> 3) & 1);
      ldmatrix_x4(b, k_tile + swz<DK>(r, c));
      mma_bf16(s[2 * np], a, b[0], b[1]);
      mma_bf16(s[2 * np + 1], a, b[2], b[3]);
    }
  }
}

// MAXT 512: blocks of more than 256 threads have 128 registers a thread; half of the Q fragments then stay in shared memory.
template <int DK, int DV, int NT, int MAXT>
__global__ void __launch_bounds__(MAXT, 1) attn_mixed_tc_kernel(MixedTcArgs a) {
  pdl_sync();
  extern __shared__ __align__(128) uint8_t smem[];
  constexpr int KT = 8 * NT, RS = KT + 8;             // keys a tile; floats a row of raw scores takes
  const int H = a.heads, G = a.kv_heads, per = H / G;
  const int hpw = a.hpw, qpw = a.qpw, wps = H / hpw, MQ = a.nsub * qpw;
  const int nwarps = blockDim.x >> 5;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = warp / wps, hb = (warp % wps) * hpw, kvh = hb / per;
  const bool split_mode = a.seq_list != nullptr;
  int seq, t0, nq, q0, pos0, lo, hi_cta, split = 0, li = 0;
  if (split_mode) {
    li = blockIdx.x, split = blockIdx.y;
    seq = a.seq_list[li];
    t0 = a.query_start[seq], nq = 1, q0 = 0;
    pos0 = a.context_lens[seq] - 1;
    lo = split * a.split_keys;
    if (lo > pos0) return;
    hi_cta = split == a.max_splits - 1 ? pos0 : min(pos0, lo + a.split_keys - 1);
  } else {
    seq = blockIdx.y;
    t0 = a.query_start[seq];
    nq = a.query_start[seq + 1] - t0;
    q0 = blockIdx.x * MQ;
    if (q0 >= nq) return;
    pos0 = a.context_lens[seq] - nq;
    lo = 0;
    hi_cta = pos0 + min(nq, q0 + MQ) - 1;
  }
  const int* table = a.block_tables + static_cast<long long>(seq) * a.max_blocks;

  // shared memory: K tiles | V tiles (first the Q tile) | raw scores | the mix | key rows of two tiles
  const int k_bytes = G * KT * DK * 2, v_bytes = G * KT * DV * 2, q_bytes = nwarps * 16 * DK * 2;
  const int second = (max(v_bytes, q_bytes) + 127) & ~127;
  const uint32_t k_buf = smem_addr(smem), v_buf = k_buf + k_bytes;
  float* raw = reinterpret_cast<float*>(smem + k_bytes + second);              // [H][MQ][RS]
  float* mixs = raw + H * MQ * RS;                                              // [H][H], times scale * log2 e
  int* rows = reinterpret_cast<int*>(mixs + H * H);                             // [2][KT]
  constexpr int KREG = MAXT > 256 ? DK / 32 : DK / 16;                          // k-steps whose Q fragments stay in registers
  const uint32_t kept = ((smem_addr(rows + 2 * KT) + 15u) & ~15u) + (warp * (DK / 16 - KREG) * 32 + lane) * 16;   // [warps][DK / 16 - KREG][32] x 16 bytes

  const int tile0 = lo / KT;
  const int n_tiles = hi_cta / KT - tile0 + 1;
  tile_rows<KT>(rows + (tile0 & 1) * KT, table, G, a.page_size, tile0 * KT, hi_cta);
  {
    constexpr int CPR = DK / 8;
    for (int id = threadIdx.x; id < nwarps * 16 * CPR; id += blockDim.x) {
      const int r = id / CPR, c = id - r * CPR;
      const int w = r >> 4, rr = r & 15;
      const int hh = (w % wps) * hpw + rr / qpw, qi = q0 + (w / wps) * qpw + rr % qpw;
      const bool valid = qi < nq;
      const __nv_bfloat16* src = a.q;
      if (valid) src = a.q + static_cast<long long>(t0 + qi) * a.q_stride + hh * DK + c * 8;
      cp_async16(v_buf + swz<DK>(r, c), src, valid ? 16 : 0);
    }
  }
  cp_async_commit();
  for (int e = threadIdx.x; e < H * H; e += blockDim.x)
    mixs[e] = (a.mix != nullptr ? a.mix[e] : (e / H == e % H ? 1.0f : 0.0f)) * a.scale_log2;
  __syncthreads();
  load_plane_tiles<DK, KT>(k_buf, a.k_cache, rows + (tile0 & 1) * KT, G, a.page_size);
  cp_async_commit();
  cp_async_wait<1>();            // Q has landed
  __syncthreads();
  uint32_t qf[KREG][4];
#pragma unroll
  for (int ks = 0; ks < DK / 16; ++ks) {
    if (ks < KREG) {
      ldmatrix_x4(qf[ks < KREG ? ks : 0], v_buf + swz<DK>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
    } else {
      uint32_t f[4];
      ldmatrix_x4(f, v_buf + swz<DK>(warp * 16 + (lane & 15), ks * 2 + (lane >> 4)));
      sts_u4(kept + (ks - KREG) * 512, f);       // read back by the same lane only
    }
  }
  __syncthreads();               // the Q tile's room becomes the V buffer
  load_plane_tiles<DV, KT>(v_buf, a.v_cache, rows + (tile0 & 1) * KT, G, a.page_size);
  cp_async_commit();

  const int gq = lane >> 2, tq = lane & 3;
  // this thread's two rows (gq and gq + 8 of the warp's 16): head hb + r / qpw, query position sub * qpw + r % qpw
  int row_lim[2];
  uint32_t my_raw[2], mix_row[2], src[2];       // shared-memory addresses: where the row's raw scores go, its row of the mix,
                                                // and head 0's raw scores of its query position
  const uint32_t raw_addr = smem_addr(raw), mix_addr = smem_addr(mixs);
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = gq + 8 * half;
    const int head = hb + r / qpw, ql = sub * qpw + r % qpw;
    const int qi = q0 + ql;
    row_lim[half] = qi < nq ? min(pos0 + qi, hi_cta) : -1;
    my_raw[half] = raw_addr + ((head * MQ + ql) * RS + tq * 2) * 4;
    mix_row[half] = mix_addr + head * H * 4;
    src[half] = raw_addr + (ql * RS + tq * 2) * 4;
  }
  int warp_hi = -1;
  {
    const int q_last = min(nq - 1, q0 + sub * qpw + qpw - 1);
    if (q0 + sub * qpw < nq) warp_hi = min(pos0 + q_last, hi_cta);
  }
  const bool with_sink = a.sink != 0 && split == 0;
  float m[2], l[2];
  m[0] = m[1] = with_sink ? 0.0f : -INFINITY;
  l[0] = l[1] = with_sink ? 1.0f : 0.0f;
  float acc[DV / 8][4];
#pragma unroll
  for (int j = 0; j < DV / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
  const uint32_t head_stride = MQ * RS * 4;

  for (int i = 0; i < n_tiles; ++i) {
    const int tile = tile0 + i;
    const int key0 = tile * KT;
    if (i + 1 < n_tiles) tile_rows<KT>(rows + ((tile + 1) & 1) * KT, table, G, a.page_size, key0 + KT, hi_cta);
    cp_async_wait<1>();          // this tile's K
    __syncthreads();
    const bool active = key0 <= warp_hi;
    float s[NT][4];
    if (active) {
#pragma unroll
      for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
      qk_rows<DK, NT, KREG>(s, qf, kept, k_buf + kvh * (KT * DK * 2));
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        sts_f2(my_raw[0] + j * 32, s[j][0], s[j][1]);
        sts_f2(my_raw[1] + j * 32, s[j][2], s[j][3]);
      }
    }
    cp_async_wait<0>();          // this tile's V
    __syncthreads();
    if (i + 1 < n_tiles) load_plane_tiles<DK, KT>(k_buf, a.k_cache, rows + ((tile + 1) & 1) * KT, G, a.page_size);
    cp_async_commit();
    if (active) {
#pragma unroll
      for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
      for (int g = 0; g < H; ++g) {
        const float w0 = lds_f(mix_row[0] + g * 4), w1 = lds_f(mix_row[1] + g * 4);
        const uint32_t p0 = src[0] + g * head_stride, p1 = src[1] + g * head_stride;
#pragma unroll
        for (int j = 0; j < NT; ++j) {
          const float2 lo2 = lds_f2(p0 + j * 32);
          const float2 hi2 = lds_f2(p1 + j * 32);
          s[j][0] = fmaf(w0, lo2.x, s[j][0]);
          s[j][1] = fmaf(w0, lo2.y, s[j][1]);
          s[j][2] = fmaf(w1, hi2.x, s[j][2]);
          s[j][3] = fmaf(w1, hi2.y, s[j][3]);
        }
      }
#pragma unroll
      for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = key0 + j * 8 + tq * 2 + (e & 1);
          if (key > row_lim[e >> 1]) s[j][e] = -INFINITY;
        }
      }
      softmax_update<DV, NT>(s, m, l, acc);
      pv_tile<DV, NT>(acc, s, v_buf + kvh * (KT * DV * 2), 0, true);
    }
    __syncthreads();
    if (i + 1 < n_tiles) load_plane_tiles<DV, KT>(v_buf, a.v_cache, rows + ((tile + 1) & 1) * KT, G, a.page_size);
    cp_async_commit();
  }
  cp_async_wait<0>();

  const int DVs = DV + 2;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = gq + 8 * half;
    const int qi = q0 + sub * qpw + r % qpw;
    if (qi >= nq) continue;
    const int h = hb + r / qpw;
    if (split_mode) {
      // the sums as they are, the maximum in natural units, the weight sum: attention_merge joins the splits
      float* dst = a.scratch + ((static_cast<long long>(li) * H + h) * a.max_splits + split) * DVs;
#pragma unroll
      for (int j = 0; j < DV / 8; ++j)
        *reinterpret_cast<float2*>(dst + j * 8 + tq * 2) = make_float2(acc[j][2 * half], acc[j][2 * half + 1]);
      if (tq == 0) {
        dst[DV] = m[half] * 0.6931471805599453f;
        dst[DV + 1] = l[half];
      }
    } else {
      const float inv = l[half] > 0.0f ? 1.0f / l[half] : 0.0f;
      __nv_bfloat16* o = a.out + (static_cast<long long>(t0 + qi) * H + h) * DV;
#pragma unroll
      for (int j = 0; j < DV / 8; ++j)
        *reinterpret_cast<uint32_t*>(o + j * 8 + tq * 2) = pack_bf16(acc[j][2 * half] * inv, acc[j][2 * half + 1] * inv);
    }
  }
}

struct MixedTcPlan {
  int hpw, qpw, nsub, nt;      // nt = 0: the kernel does not take the geometry
  size_t smem;
};

static int gcd_int(int a, int b) { return b == 0 ? a : gcd_int(b, a % b); }

// Shared memory of a block: K tiles, V tiles (or the Q tile if larger), raw scores, the mix, key rows of two tiles, and
// for blocks of more than 8 warps half of the Q fragments.
static size_t mixed_tc_smem(int heads, int kv_heads, int dim, int vdim, int warps, int mq, int kt) {
  const size_t k = static_cast<size_t>(kv_heads) * kt * dim * 2, v = static_cast<size_t>(kv_heads) * kt * vdim * 2;
  const size_t q = static_cast<size_t>(warps) * 16 * dim * 2;
  const size_t second = ((v > q ? v : q) + 127) / 128 * 128;
  const size_t kept = warps > 8 ? static_cast<size_t>(warps) * (dim / 32) * 512 + 16 : 0;      // Q fragments that leave the registers, on 16 bytes
  return k + second + static_cast<size_t>(heads) * mq * (kt + 8) * 4 + static_cast<size_t>(heads) * heads * 4 + 2 * kt * 4 + kept;
}

constexpr size_t kMixedTcSmemLimit = 208 * 1024;
constexpr int kMixedTcMaxWarps = 16;

// The warp shape, the groups of query positions a block (prompts: as many as 16 warps and 64 positions allow; single
// rows: one) and the largest key tile that fits shared memory; tiles of 16 keys only when no larger one fits at all.
static MixedTcPlan mixed_tc_plan(int heads, int kv_heads, int dim, int vdim, bool single) {
  MixedTcPlan p{0, 0, 0, 0, 0};
  if (!((dim == 64 || dim == 128) && (vdim == 64 || vdim == 128)) || heads <= 0 || kv_heads <= 0 || heads % kv_heads != 0) return p;
  p.hpw = gcd_int(heads / kv_heads, 16);
  p.qpw = 16 / p.hpw;
  const int wps = heads / p.hpw;
  if (wps > kMixedTcMaxWarps) return p;
  int most = kMixedTcMaxWarps / wps;
  if (most > 64 / p.qpw) most = 64 / p.qpw;
  if (single || most < 1) most = 1;
  for (int min_nt = 4; min_nt >= 2; min_nt -= 2)
    for (int nsub = most; nsub >= 1; --nsub)
      for (int nt = 8; nt >= min_nt; nt /= 2) {
        if (nt == 8 && wps * nsub > 8) continue;      // 64 keys a tile need more registers than 512 threads leave
        const size_t smem = mixed_tc_smem(heads, kv_heads, dim, vdim, wps * nsub, nsub * p.qpw, 8 * nt);
        if (smem <= kMixedTcSmemLimit) {
          p.nsub = nsub, p.nt = nt, p.smem = smem;
          return p;
        }
      }
  return p;
}

template <int DK, int DV>
static int launch_mixed_tc(const MixedTcArgs& a, dim3 grid, const MixedTcPlan& p, cudaStream_t s) {
  const int threads = 32 * (a.heads / p.hpw) * p.nsub;
#define TIE_MIXED_TC_CASE(NT, MAXT)                                                                           \
  do {                                                                                                        \
    cudaFuncSetAttribute(attn_mixed_tc_kernel<DK, DV, NT, MAXT>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                         static_cast<int>(p.smem));                                                           \
    TIE_LAUNCH((attn_mixed_tc_kernel<DK, DV, NT, MAXT>), grid, threads, p.smem, s, a);                        \
  } while (0)
  if (threads <= 256) {
    if (p.nt == 8) TIE_MIXED_TC_CASE(8, 256);
    else if (p.nt == 4) TIE_MIXED_TC_CASE(4, 256);
    else TIE_MIXED_TC_CASE(2, 256);
  } else {
    if (p.nt == 4) TIE_MIXED_TC_CASE(4, 512);
    else TIE_MIXED_TC_CASE(2, 512);
  }
#undef TIE_MIXED_TC_CASE
  TIE_RETURN_LAUNCH("attention_mixed_tc");
}

}  // namespace tie

using namespace tie;

// 1 when tie_attention_mixed_tc takes this geometry (bfloat16 only), else 0.
TIE_API int tie_attention_mixed_tc_takes(int heads, int kv_heads, int dim, int vdim) {
  return mixed_tc_plan(heads, kv_heads, dim, vdim, false).nt > 0 && mixed_tc_plan(heads, kv_heads, dim, vdim, true).nt > 0 ? 1 : 0;
}

// Prompts (seq_list null): sequences 0 .. n_seqs-1 of the step each bring several tokens, at most max_queries. Single
// rows: one row per sequence of seq_list [n_seqs], keys in splits of split_keys (a multiple of 64) whose (sums,
// maximum, weight sum) go to scratch [n_seqs, heads, max_splits, vdim + 2] for tie_attention_merge.
TIE_API int tie_attention_mixed_tc(const void* q, long long q_stride, const void* k_cache, const void* v_cache, void* out,
                                   const float* mix, const int* query_start, const int* context_lens, const int* block_tables,
                                   int max_blocks, int n_seqs, int max_queries, int heads, int kv_heads, int dim, int vdim,
                                   int page_size, float scale, int sink, const int* seq_list, int split_keys, int max_splits,
                                   float* scratch, cudaStream_t s) {
  TIE_REQUIRE(heads > 0 && kv_heads > 0 && page_size > 0 && n_seqs >= 0 && max_queries >= 0, "attention_mixed_tc: bad sizes");
  const bool single = seq_list != nullptr;
  const MixedTcPlan p = mixed_tc_plan(heads, kv_heads, dim, vdim, single);
  TIE_REQUIRE(p.nt > 0, "attention_mixed_tc: heads=%d kv_heads=%d dim=%d vdim=%d is served by the CUDA-core kernel", heads, kv_heads,
              dim, vdim);
  TIE_REQUIRE(q_stride % 8 == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0, "attention_mixed_tc: q rows must start on 16 bytes");
  TIE_REQUIRE(!single || (split_keys > 0 && split_keys % 64 == 0 && max_splits > 0 && scratch != nullptr),
              "attention_mixed_tc: splits of a multiple of 64 keys and their scratch, got %d", split_keys);
  if (n_seqs == 0 || (!single && max_queries == 0)) return kOk;
  MixedTcArgs a{};
  a.q = static_cast<const __nv_bfloat16*>(q), a.q_stride = q_stride;
  a.k_cache = static_cast<const __nv_bfloat16*>(k_cache), a.v_cache = static_cast<const __nv_bfloat16*>(v_cache);
  a.out = static_cast<__nv_bfloat16*>(out), a.mix = mix;
  a.query_start = query_start, a.context_lens = context_lens, a.block_tables = block_tables;
  a.max_blocks = max_blocks, a.heads = heads, a.kv_heads = kv_heads, a.page_size = page_size;
  a.hpw = p.hpw, a.qpw = p.qpw, a.nsub = p.nsub;
  a.scale_log2 = scale * 1.4426950408889634f, a.sink = sink;
  a.seq_list = seq_list, a.split_keys = split_keys, a.max_splits = max_splits, a.scratch = scratch;
  const dim3 grid = single ? dim3(n_seqs, max_splits) : dim3(ceil_div(max_queries, p.nsub * p.qpw), n_seqs);
  if (dim == 64 && vdim == 64) return launch_mixed_tc<64, 64>(a, grid, p, s);
  if (dim == 64 && vdim == 128) return launch_mixed_tc<64, 128>(a, grid, p, s);
  if (dim == 128 && vdim == 64) return launch_mixed_tc<128, 64>(a, grid, p, s);
  return launch_mixed_tc<128, 128>(a, grid, p, s);
}
