// The gated delta rule with one decay per key channel, as a recurrence over the tokens of each sequence.
//
// Per value head, a float matrix S (key channels x value channels) is carried from token to token:
//
//     S <- diag(decay_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//
// (the read-out sees the token's own write). q_t and k_t are unit vectors per head (q also scaled), made from
// projections that pass a short causal convolution over time and SiLU; decay_t = exp(-rate_h softplus(a_t + bias))
// per key channel. Columns of S do not depend on one another, so the work is cut by (sequence, head, columns).
//
// Three kernels, all of them float inside:
//   delta_prep   one block per (token, head of q, k or v): convolution (its first taps - 1 inputs come from the
//                sequence's state slot or from the rows ahead of it in the step) + SiLU, unit norm of q and k per
//                head; further blocks turn the raw decay projection into decays (in place) and take beta's sigmoid.
//   delta_rule   one block per (sequence, head, 16 columns): the recurrence over the sequence's tokens of the
//                step, state read from and written back to the slot in row pieces through shared memory. Eight
//                lanes share a column, each holding every eighth key channel; a chunk of tokens is staged in shared
//                memory at a time. The blocks of a sequence also move the convolution's last inputs into the
//                slot, a slice of the channels each.
//   delta_out    one warp per (token, head): o / rms(o) * w * sigmoid(gate).
//
// A state slot is one float row: S of every head [heads, dim, vdim], then the convolution's last taps - 1
// inputs [taps - 1, channels] (oldest first), channels = q, k, v one after the other.
#include <math.h>

#include "common.cuh"

namespace tie {

struct DeltaShape {
  int heads, kv_heads, dim, vdim, taps;
  int channels() const { return 2 * kv_heads * dim + heads * vdim; }
};

__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.0f ? z : log1pf(expf(z)); }

// proj row: q at q_off [kv_heads * dim], k at k_off, v at v_off [heads * vdim], beta at b_off [heads].
// One block per (token, unit). Units: the q heads, the k heads, the v heads (convolution + SiLU over the unit's
// channels; q and k also their unit norm), then one unit per head that turns the raw decay projection into decays
// in place, and a last one for beta.
template <typename T>
__global__ void __launch_bounds__(128) delta_prep_kernel(const T* __restrict__ proj, long long stride, int q_off, int k_off,
                                                         int v_off, int b_off, const float* __restrict__ conv_w,
                                                         const float* __restrict__ state, long long state_stride,
                                                         long long conv_state_off, const int* __restrict__ seq_of_row,
                                                         const int* __restrict__ query_start,
                                                         const int* __restrict__ state_slots, DeltaShape sh, float unit_eps,
                                                         float q_scale, float* __restrict__ qn, float* __restrict__ kn,
                                                         float* __restrict__ vn, float* __restrict__ beta,
                                                         float* __restrict__ decay, long long decay_stride,
                                                         const float* __restrict__ dt_bias, const float* __restrict__ a_log) {
  pdl_sync();
  __shared__ float scratch[33];
  const int t = blockIdx.x, unit = blockIdx.y;
  const int G = sh.kv_heads, H = sh.heads, dim = sh.dim, vdim = sh.vdim, taps = sh.taps;
  const int nqk = G * dim, nv = H * vdim, C = 2 * nqk + nv;
  const T* row = proj + static_cast<long long>(t) * stride;
  if (unit == 2 * G + 2 * H) {
    for (int h = threadIdx.x; h < H; h += blockDim.x) beta[static_cast<long long>(t) * H + h] = sigmoidf_(ld(row + b_off + h));
    return;
  }
  if (unit >= 2 * G + H) {            // decay = exp(-rate * softplus(raw + bias)), in place
    const int h = unit - (2 * G + H);
    const float rate = expf(a_log[h]);
    float* a = decay + static_cast<long long>(t) * decay_stride + h * dim;
    for (int d = threadIdx.x; d < dim; d += blockDim.x) a[d] = expf(-rate * softplusf_(a[d] + dt_bias[h * dim + d]));
    return;
  }
  const int s = seq_of_row[t];
  const int j = t - query_start[s];          // tokens of this sequence ahead of this one in the step
  const int slot = state_slots[s];
  const float* tail = slot >= 0 ? state + slot * state_stride + conv_state_off : nullptr;
  const bool is_v = unit >= 2 * G;
  const int width = is_v ? vdim : dim;
  const int c0 = is_v ? 2 * nqk + (unit - 2 * G) * vdim : unit * dim;      // the unit's first channel of all C
  float* dst = is_v ? vn + static_cast<long long>(t) * nv + (unit - 2 * G) * vdim
                    : (unit < G ? qn + static_cast<long long>(t) * nqk + unit * dim
                                : kn + static_cast<long long>(t) * nqk + (unit - G) * dim);
  float vals[2] = {0.0f, 0.0f};              // dim <= 256: at most two channels of a q or k head per thread
  float ss = 0.0f;
  for (int d = threadIdx.x, n = 0; d < width; d += blockDim.x, ++n) {
    const int c = c0 + d;
    const int col = c < nqk ? q_off + c : (c < 2 * nqk ? k_off + (c - nqk) : v_off + (c - 2 * nqk));
    float y = 0.0f;
    for (int i = 0; i < taps; ++i) {
      const int back = taps - 1 - i;         // this tap's input is `back` tokens ahead of the current one
      float in;
      if (back <= j) in = ld(row - static_cast<long long>(back) * stride + col);
      else in = tail ? tail[static_cast<long long>(j + i) * C + c] : 0.0f;
      y = fmaf(conv_w[c * taps + i], in, y);
    }
    y = y * sigmoidf_(y);
    if (is_v) {
      dst[d] = y;
    } else {
      if (n < 2) vals[n] = y;
      ss += y * y;
    }
  }
  if (is_v) return;
  ss = block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss + unit_eps);
  for (int d = threadIdx.x, n = 0; d < width && n < 2; d += blockDim.x, ++n) dst[d] = unit < G ? (vals[n] * inv) * q_scale : vals[n] * inv;
}

__device__ __forceinline__ void async_copy4(float* dst, const float* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src) : "memory");
}
__device__ __forceinline__ void async_copy16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))), "l"(src) : "memory");
}
__device__ __forceinline__ void async_copies_done() { asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory"); }

constexpr int kDeltaCols = 16;       // columns of S that a block holds (LANES threads each)
constexpr int kDeltaPad = kDeltaCols + 1;

// The key channel that register r of lane `lane` (of the LANES that share a column) holds: four channels in a row,
// then the next four 32 channels on, so that a lane reads its k, q and decay entries 16 bytes at a time.
template <int LANES>
__device__ __forceinline__ int delta_row(int r, int lane) { return (r >> 2) * (4 * LANES) + lane * 4 + (r & 3); }

// One block per (sequence, head, 16 columns of S). A column's key channels are spread over LANES lanes of a warp
// (8, 16 or 32, by the head size: more lanes mean more warps to hide each other's latencies and fewer registers
// each), so a token costs one pass over the registers with two dot products (against k and
// against q of the decayed state, and k . q beside them), three shuffle steps for the three, and the update: with
// d1 = (gS)^T k and d2 = (gS)^T q, u = beta (v - d1) and the read-out of the updated state is o = d2 + (k . q) u.
// RMAX: key channels a lane may hold (dim <= LANES * RMAX).
// BONUS (a specialization of the plain mode): the token reads the state as the token before left it and sees its own
// write through a weight per key channel, o = S^T q + (sum_c bonus[h, c] k_c q_c) u, and only then S <- diag(decay) S + k u^T.
template <typename T, int RMAX, int LANES, bool PLAIN, bool BONUS = false>
__global__ void __launch_bounds__(LANES * kDeltaCols) delta_rule_kernel(
    const float* __restrict__ qn, const float* __restrict__ kn, const float* __restrict__ vn, const float* __restrict__ beta,
    const float* __restrict__ decay, long long decay_stride, float* __restrict__ state, long long state_stride,
    long long conv_state_off, const T* __restrict__ proj, long long proj_stride, int q_off, int k_off, int v_off,
    const int* __restrict__ query_start, const int* __restrict__ state_slots, DeltaShape sh, int chunk,
    float* __restrict__ out, int decay_per_head, const float* __restrict__ bonus = nullptr) {
  // A block is one long chain of dependent steps, and there are few blocks (sequences x heads x column tiles). Started early
  // (programmatic dependent launch), beside a kernel that still fills the GPU, the blocks were placed on the few SMs that had
  // room first and shared them: 1.7 instead of 0.6 ms for 2,048 tokens. So the launcher starts this kernel only when the
  // kernels ahead have drained (launch_kernel_alone), and the kernel behind is let in when the walk over the tokens is done.
  pdl_wait();
  extern __shared__ float smem[];
  const int s = blockIdx.x, h = blockIdx.y, col0 = blockIdx.z * kDeltaCols;
  const int slot = state_slots[s];
  if (slot < 0) return;                       // a sequence that pads a captured batch
  const int t0 = query_start[s], n = query_start[s + 1] - t0;
  const int dim = sh.dim, vdim = sh.vdim, nqk = sh.kv_heads * dim, nv = sh.heads * vdim;
  const int g = h / (sh.heads / sh.kv_heads);
  const int lane8 = threadIdx.x % LANES, cidx = threadIdx.x / LANES, col = col0 + cidx;      // lane8: the lane among those of its column
  const bool live = col < vdim;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* S = state + slot * state_stride + static_cast<long long>(h) * dim * vdim;
  // The block's 16 columns of S come in row pieces of 64 bytes through shared memory (the lanes' own elements
  // are a row apart in memory).
  for (int i = threadIdx.x; i < dim * kDeltaCols; i += blockDim.x) {
    const int r = i / kDeltaCols, c = i % kDeltaCols;
    smem[r * kDeltaPad + c] = col0 + c < vdim ? S[static_cast<long long>(r) * vdim + col0 + c] : 0.0f;
  }
  __syncthreads();
  float sreg[RMAX];
#pragma unroll
  for (int r = 0; r < RMAX; ++r) {
    const int rowi = delta_row<LANES>(r, lane8);
    sreg[r] = rowi < dim ? smem[rowi * kDeltaPad + cidx] : 0.0f;
  }
  // Chunks of tokens come through two buffers in turn: while one is worked on, asynchronous copies fill the other.
  // A buffer: k [chunk][dim], q [chunk][dim], decays [chunk][dim], v [chunk][kDeltaCols], beta [chunk].
  const int buf_floats = (chunk * (3 * dim + kDeltaCols + 1) + 3) & ~3;      // a buffer starts on a 16-byte boundary
  const bool vec4 = dim % 4 == 0;
  const bool wide = !decay_per_head && vec4 && nqk % 4 == 0 && decay_stride % 4 == 0 && ((reinterpret_cast<uintptr_t>(kn) | reinterpret_cast<uintptr_t>(qn) |
                                                                      reinterpret_cast<uintptr_t>(decay)) & 15) == 0;
  auto fetch = [&](int c0, float* base) {
    const int cn = min(chunk, n - c0);
    float* kb = base;
    float* qb = kb + chunk * dim;
    float* gb = qb + chunk * dim;
    float* vb = gb + chunk * dim;
    float* bb = vb + chunk * kDeltaCols;
    if (wide) {
      const int pieces = dim / 4;
      for (int i = threadIdx.x; i < cn * pieces; i += blockDim.x) {
        const int tc = i / pieces, d = (i % pieces) * 4;
        const long long t = t0 + c0 + tc;
        async_copy16(kb + tc * dim + d, kn + t * nqk + g * dim + d);
        async_copy16(qb + tc * dim + d, qn + t * nqk + g * dim + d);
        async_copy16(gb + tc * dim + d, decay + t * decay_stride + h * dim + d);
      }
    } else {
      for (int i = threadIdx.x; i < cn * dim; i += blockDim.x) {
        const int tc = i / dim, d = i % dim;
        const long long t = t0 + c0 + tc;
        async_copy4(kb + i, kn + t * nqk + g * dim + d);
        async_copy4(qb + i, qn + t * nqk + g * dim + d);
        async_copy4(gb + i, decay + t * decay_stride + (decay_per_head ? h : h * dim + d));
      }
    }
    for (int i = threadIdx.x; i < cn * kDeltaCols; i += blockDim.x) {
      const int tc = i / kDeltaCols, c = col0 + i % kDeltaCols;
      if (c < vdim) async_copy4(vb + i, vn + (t0 + c0 + tc) * static_cast<long long>(nv) + h * vdim + c);
      else vb[i] = 0.0f;
    }
    for (int i = threadIdx.x; i < cn; i += blockDim.x) {
      if (beta) async_copy4(bb + i, beta + (t0 + c0 + i) * static_cast<long long>(sh.heads) + h);
      else bb[i] = 1.0f;
    }
  };
  __syncthreads();                            // the staging tile above is done with: the buffers lie over it
  fetch(0, smem);
  int turn = 0;
  for (int c0 = 0; c0 < n; c0 += chunk, turn ^= 1) {
    const int cn = min(chunk, n - c0);
    float* base = smem + turn * buf_floats;
    const float* kb = base;
    const float* qb = kb + chunk * dim;
    const float* gb = qb + chunk * dim;
    const float* vb = gb + chunk * dim;
    const float* bb = vb + chunk * kDeltaCols;
    async_copies_done();
    __syncthreads();                          // this chunk is there, and everyone is through with the other buffer
    if (c0 + chunk < n) fetch(c0 + chunk, smem + (turn ^ 1) * buf_floats);
    float* kq = smem + 2 * buf_floats;        // [chunk <= 16]
    if (PLAIN) {
      // k . q of a token is the same for every column: once a chunk, a warp a token, instead of once a column
      for (int tc = warp; tc < cn; tc += static_cast<int>(blockDim.x >> 5)) {
        float dot = 0.0f;
        for (int d = lane; d < dim; d += 32)
          dot = fmaf(BONUS ? kb[tc * dim + d] * bonus[h * dim + d] : kb[tc * dim + d], qb[tc * dim + d], dot);
        dot = warp_sum(dot);
        if (lane == 0) kq[tc] = dot;
      }
      __syncthreads();
    }
    for (int tc = 0; tc < cn; ++tc) {
      const float* kt = kb + tc * dim;
      const float* qt = qb + tc * dim;
      const float* gt = gb + tc * dim;
      float kreg[RMAX];
      float d1a = 0.0f, d1b = 0.0f, d2a = 0.0f, d2b = 0.0f, d3 = 0.0f;     // d3: k . q over this lane's channels
#pragma unroll
      for (int q4 = 0; q4 < RMAX / 4; ++q4) {
        const int r0 = delta_row<LANES>(4 * q4, lane8);
        float kk[4], qq[4], gg[4];
        if (vec4) {                              // dim % 4 == 0: the lane's four channels are one 16-byte piece
          if (r0 < dim) {
            const float4 k4 = *reinterpret_cast<const float4*>(kt + r0), q4v = *reinterpret_cast<const float4*>(qt + r0),
                         g4 = *reinterpret_cast<const float4*>(gt + r0);
            kk[0] = k4.x, kk[1] = k4.y, kk[2] = k4.z, kk[3] = k4.w;
            qq[0] = q4v.x, qq[1] = q4v.y, qq[2] = q4v.z, qq[3] = q4v.w;
            gg[0] = g4.x, gg[1] = g4.y, gg[2] = g4.z, gg[3] = g4.w;
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) kk[e] = qq[e] = gg[e] = 0.0f;
          }
        } else {
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const bool in = r0 + e < dim;
            kk[e] = in ? kt[r0 + e] : 0.0f;
            qq[e] = in ? qt[r0 + e] : 0.0f;
            gg[e] = in ? gt[r0 + e] : 0.0f;
          }
        }
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float s0 = sreg[4 * q4 + e];
          const float sv = s0 * gg[e];
          const float seen = BONUS ? s0 : sv;     // what the read-out sees of the state: before or after the decay
          sreg[4 * q4 + e] = sv;
          kreg[4 * q4 + e] = kk[e];
          if (e & 1) {
            if (!PLAIN) d1b = fmaf(kk[e], sv, d1b);
            d2b = fmaf(qq[e], seen, d2b);
          } else {
            if (!PLAIN) d1a = fmaf(kk[e], sv, d1a);
            d2a = fmaf(qq[e], seen, d2a);
          }
          if (!PLAIN) d3 = fmaf(kk[e], qq[e], d3);
        }
      }
      float d1 = d1a + d1b, d2 = d2a + d2b;
#pragma unroll
      for (int o = 1; o < LANES; o <<= 1) {
        if (!PLAIN) d1 += __shfl_xor_sync(0xffffffffu, d1, o);
        d2 += __shfl_xor_sync(0xffffffffu, d2, o);
        if (!PLAIN) d3 += __shfl_xor_sync(0xffffffffu, d3, o);
      }
      const float u = PLAIN ? bb[tc] * vb[tc * kDeltaCols + cidx] : bb[tc] * (vb[tc * kDeltaCols + cidx] - d1);
      if (PLAIN) d3 = kq[tc];
      if (live && lane8 == 0) out[(t0 + c0 + tc) * static_cast<long long>(nv) + h * vdim + col] = fmaf(d3, u, d2);
#pragma unroll
      for (int r = 0; r < RMAX; ++r) sreg[r] = fmaf(kreg[r], u, sreg[r]);
    }
  }
  pdl_launch_dependents();
  __syncthreads();
#pragma unroll
  for (int r = 0; r < RMAX; ++r) {
    const int rowi = delta_row<LANES>(r, lane8);
    if (rowi < dim) smem[rowi * kDeltaPad + cidx] = sreg[r];
  }
  __syncthreads();
  for (int i = threadIdx.x; i < dim * kDeltaCols; i += blockDim.x) {
    const int r = i / kDeltaCols, c = i % kDeltaCols;
    if (col0 + c < vdim) S[static_cast<long long>(r) * vdim + col0 + c] = smem[r * kDeltaPad + c];
  }
  // The convolution's last taps - 1 inputs after this step: from the step's rows where it brought enough, else
  // what the slot held moves up. Every block of the sequence takes a slice of the channels.
  if (sh.taps > 1) {
    const int C = 2 * nqk + nv, keep = sh.taps - 1;
    const int blocks = gridDim.y * gridDim.z, mine = blockIdx.y * gridDim.z + blockIdx.z;
    const int per = (C + blocks - 1) / blocks;
    const int c_end = min(C, (mine + 1) * per);
    float* tail = state + slot * state_stride + conv_state_off;
    for (int c = mine * per + threadIdx.x; c < c_end; c += blockDim.x) {
      const int pc = c < nqk ? q_off + c : (c < 2 * nqk ? k_off + (c - nqk) : v_off + (c - 2 * nqk));
      for (int i = 0; i < keep; ++i) {
        const int from = n - keep + i;        // offset in the step of the token that lands at place i
        tail[static_cast<long long>(i) * C + c] = from >= 0 ? ld(proj + (t0 + from) * proj_stride + pc)
                                                            : tail[static_cast<long long>(n + i) * C + c];
      }
    }
  }
}

template <typename T>
__global__ void __launch_bounds__(128) delta_out_kernel(const float* __restrict__ o, const float* __restrict__ gate,
                                                        long long gate_stride, const float* __restrict__ w, float eps,
                                                        T* __restrict__ out, int heads, int vdim, long long items) {
  pdl_sync();
  const int lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= items) return;
  const long long t = item / heads;
  const int h = static_cast<int>(item % heads);
  const float* x = o + item * vdim;
  float ss = 0.0f;
  for (int d = lane; d < vdim; d += 32) ss += x[d] * x[d];
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(vdim) + eps);
  for (int d = lane; d < vdim; d += 32)
    st(out + item * vdim + d, ((x[d] * inv) * w[d]) * sigmoidf_(gate[t * gate_stride + h * vdim + d]));
}

}  // namespace tie

using namespace tie;

static int check_delta(const DeltaShape& sh) {
  TIE_REQUIRE(sh.heads > 0 && sh.kv_heads > 0 && sh.heads % sh.kv_heads == 0 && sh.dim > 0 && sh.dim <= 256 && sh.vdim > 0 &&
                  sh.taps >= 1 && sh.taps <= 16,
              "delta rule: bad shape heads=%d/%d dim=%d (1 to 256) vdim=%d taps=%d (1 to 16)", sh.heads, sh.kv_heads, sh.dim,
              sh.vdim, sh.taps);
  return kOk;
}

TIE_API int tie_delta_prep(int dtype, const void* proj, long long stride, int q_off, int k_off, int v_off, int b_off,
                           const float* conv_w, const float* state, long long state_stride, long long conv_state_off,
                           const int* seq_of_row, const int* query_start, const int* state_slots, int tokens, int heads,
                           int kv_heads, int dim, int vdim, int taps, float unit_eps, float q_scale, float* qn, float* kn,
                           float* vn, float* beta, float* decay, long long decay_stride, const float* dt_bias,
                           const float* a_log, cudaStream_t s) {
  const DeltaShape sh{heads, kv_heads, dim, vdim, taps};
  if (const int st_ = check_delta(sh)) return st_;
  if (tokens <= 0) return kOk;
  const int units = 2 * kv_heads + 2 * heads + 1;
  TIE_REQUIRE(units <= 65535, "delta_prep: %d heads exceed the grid", heads);
  const dim3 grid(tokens, units);
  if (dtype == TIE_F32) {
    TIE_LAUNCH((delta_prep_kernel<float>), grid, 128, 0, s, static_cast<const float*>(proj), stride, q_off, k_off, v_off, b_off,
               conv_w, state, state_stride, conv_state_off, seq_of_row, query_start, state_slots, sh, unit_eps, q_scale, qn, kn,
               vn, beta, decay, decay_stride, dt_bias, a_log);
  } else if (dtype == TIE_BF16) {
    TIE_LAUNCH((delta_prep_kernel<__nv_bfloat16>), grid, 128, 0, s, static_cast<const __nv_bfloat16*>(proj), stride, q_off,
               k_off, v_off, b_off, conv_w, state, state_stride, conv_state_off, seq_of_row, query_start, state_slots, sh,
               unit_eps, q_scale, qn, kn, vn, beta, decay, decay_stride, dt_bias, a_log);
  } else {
    set_error("unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("delta_prep");
}

template <typename T>
static int launch_delta_rule(const float* qn, const float* kn, const float* vn, const float* beta, const float* decay,
                             long long decay_stride, float* state, long long state_stride, long long conv_state_off,
                             const void* proj, long long proj_stride, int q_off, int k_off, int v_off,
                             const int* query_start, const int* state_slots, int seqs, const DeltaShape& sh, float* out,
                             int plain, int decay_per_head, cudaStream_t s, const float* bonus = nullptr) {
  const dim3 grid(seqs, sh.heads, ceil_div(sh.vdim, kDeltaCols));
  const int per_token = 3 * sh.dim + kDeltaCols + 1;
  int chunk = (44 * 1024 / static_cast<int>(sizeof(float))) / (2 * per_token);      // two buffers
  chunk = chunk > 16 ? 16 : (chunk < 1 ? 1 : chunk);
  const int stage = sh.dim * kDeltaPad;                         // the state tile on its way in and out
  const int buffers = 2 * ((chunk * per_token + 3) & ~3) + 16;        // and a chunk's k . q (the plain mode)
  const int floats = buffers > stage ? buffers : stage;
  const size_t smem = static_cast<size_t>(floats) * sizeof(float);
  const T* p = static_cast<const T*>(proj);
#define TIE_DELTA_CASE(R, LANES)                                                                                          \
  do {                                                                                                                    \
    if (plain && bonus)                                                                                                   \
      tie::launch_kernel_alone(delta_rule_kernel<T, R, LANES, true, true>, grid, dim3(LANES * kDeltaCols), smem, s, qn, kn, vn, beta, decay, \
                         decay_stride, state, state_stride, conv_state_off, p, proj_stride, q_off, k_off, v_off, query_start,   \
                         state_slots, sh, chunk, out, decay_per_head, bonus);                                             \
    else if (plain)                                                                                                       \
      tie::launch_kernel_alone(delta_rule_kernel<T, R, LANES, true>, grid, dim3(LANES * kDeltaCols), smem, s, qn, kn, vn, beta, decay, \
                         decay_stride, state, state_stride, conv_state_off, p, proj_stride, q_off, k_off, v_off, query_start,   \
                         state_slots, sh, chunk, out, decay_per_head, nullptr);                                           \
    else                                                                                                                  \
      tie::launch_kernel_alone(delta_rule_kernel<T, R, LANES, false>, grid, dim3(LANES * kDeltaCols), smem, s, qn, kn, vn, beta, decay, \
                         decay_stride, state, state_stride, conv_state_off, p, proj_stride, q_off, k_off, v_off, query_start,   \
                         state_slots, sh, chunk, out, decay_per_head, nullptr);                                           \
  } while (0)
  if (sh.dim <= 32) TIE_DELTA_CASE(4, 8);
  else if (sh.dim <= 64) TIE_DELTA_CASE(4, 16);
  else if (sh.dim <= 128) TIE_DELTA_CASE(4, 32);
  else TIE_DELTA_CASE(8, 32);
#undef TIE_DELTA_CASE
  TIE_RETURN_LAUNCH("delta_rule");
}

TIE_API int tie_delta_rule(int dtype, const float* qn, const float* kn, const float* vn, const float* beta,
                           const float* decay, long long decay_stride, float* state, long long state_stride,
                           long long conv_state_off, const void* proj, long long proj_stride, int q_off, int k_off,
                           int v_off, const int* query_start, const int* state_slots, int seqs, int heads, int kv_heads,
                           int dim, int vdim, int taps, float* out, int plain, int decay_per_head, cudaStream_t s) {
  const DeltaShape sh{heads, kv_heads, dim, vdim, taps};
  if (const int st_ = check_delta(sh)) return st_;
  if (seqs <= 0) return kOk;
  TIE_REQUIRE(beta != nullptr || plain, "delta_rule: the delta rule needs beta");
  TIE_REQUIRE(seqs <= 65535 * 32 && heads <= 65535, "delta_rule: %d sequences x %d heads exceed the grid", seqs, heads);
  if (dtype == TIE_F32)
    return launch_delta_rule<float>(qn, kn, vn, beta, decay, decay_stride, state, state_stride, conv_state_off, proj, proj_stride,
                                    q_off, k_off, v_off, query_start, state_slots, seqs, sh, out, plain, decay_per_head, s);
  if (dtype == TIE_BF16)
    return launch_delta_rule<__nv_bfloat16>(qn, kn, vn, beta, decay, decay_stride, state, state_stride, conv_state_off, proj,
                                            proj_stride, q_off, k_off, v_off, query_start, state_slots, seqs, sh, out, plain, decay_per_head, s);
  set_error("unknown dtype code %d", dtype);
  return kBadArgument;
}

TIE_API int tie_delta_out(int dtype, const float* o, const float* gate, long long gate_stride, const float* w, float eps,
                          void* out, int tokens, int heads, int vdim, cudaStream_t s) {
  TIE_REQUIRE(tokens >= 0 && heads > 0 && vdim > 0, "delta_out: bad sizes tokens=%d heads=%d vdim=%d", tokens, heads, vdim);
  const long long items = static_cast<long long>(tokens) * heads;
  if (items == 0) return kOk;
  if (dtype == TIE_F32) {
    TIE_LAUNCH((delta_out_kernel<float>), ceil_div(items, 4), 128, 0, s, o, gate, gate_stride, w, eps, static_cast<float*>(out), heads,
               vdim, items);
  } else if (dtype == TIE_BF16) {
    TIE_LAUNCH((delta_out_kernel<__nv_bfloat16>), ceil_div(items, 4), 128, 0, s, o, gate, gate_stride, w, eps,
               static_cast<__nv_bfloat16*>(out), heads, vdim, items);
  } else {
    set_error("unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("delta_out");
}

// The plain recurrence read before it is written, with a weight per head and key channel on the token's own write
// (`bonus`, float [heads * dim]): o_t = (S + diag(bonus) k_t u_t^T)^T q_t, then S <- diag(decay_t) S + k_t u_t^T.
TIE_API int tie_delta_rule_bonus(int dtype, const float* qn, const float* kn, const float* vn, const float* beta,
                                 const float* decay, long long decay_stride, float* state, long long state_stride,
                                 long long conv_state_off, const void* proj, long long proj_stride, int q_off, int k_off,
                                 int v_off, const int* query_start, const int* state_slots, int seqs, int heads,
                                 int kv_heads, int dim, int vdim, int taps, float* out, const float* bonus, cudaStream_t s) {
  const DeltaShape sh{heads, kv_heads, dim, vdim, taps};
  if (const int st_ = check_delta(sh)) return st_;
  if (seqs <= 0) return kOk;
  TIE_REQUIRE(bonus != nullptr && heads == kv_heads, "delta_rule_bonus: a weight per head and key channel, and a key head per head");
  TIE_REQUIRE(seqs <= 65535 * 32 && heads <= 65535, "delta_rule: %d sequences x %d heads exceed the grid", seqs, heads);
  if (dtype == TIE_F32)
    return launch_delta_rule<float>(qn, kn, vn, beta, decay, decay_stride, state, state_stride, conv_state_off, proj, proj_stride,
                                    q_off, k_off, v_off, query_start, state_slots, seqs, sh, out, 1, 0, s, bonus);
  if (dtype == TIE_BF16)
    return launch_delta_rule<__nv_bfloat16>(qn, kn, vn, beta, decay, decay_stride, state, state_stride, conv_state_off, proj,
                                            proj_stride, q_off, k_off, v_off, query_start, state_slots, seqs, sh, out, 1, 0, s, bonus);
  set_error("unknown dtype code %d", dtype);
  return kBadArgument;
}
