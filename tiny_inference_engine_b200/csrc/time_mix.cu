// What stands around the plain recurrence (delta_rule.cu, read-first mode) for a mixer that blends every input with
// the token before:
//
//   token_shift_mix   out[s][t] = h[t] + (h[t - 1] - h[t]) * mu[s] for each of n_mix blends; the row before the first
//                     row of a sequence's portion is the one its state slot keeps (zeros at position 0).
//   tanh_rows         float rows -> tanh in the compute type (the inner activation of a two-step projection)
//   time_mix_prep     r, k, v (compute type) -> float rows; decay = exp(-exp(z + w0)) in place, float
//   time_mix_out      (o / rms(o) per head) * w[h, :] * silu(gate) in the compute type; the sequence's last row of h
//                     becomes the row that its slot keeps
#include <math.h>

#include "common.cuh"

namespace tie {

template <typename T>
__global__ void __launch_bounds__(256) token_shift_mix_kernel(const T* __restrict__ h, const float* __restrict__ mu, int n_mix,
                                                              const float* __restrict__ state, long long state_stride,
                                                              long long prev_off, const int* __restrict__ seq_of_row,
                                                              const int* __restrict__ query_start,
                                                              const int* __restrict__ positions, const int* __restrict__ state_slots,
                                                              T* __restrict__ out, long long out_stride, int D) {
  pdl_sync();
  const long long t = blockIdx.x;
  const int s = seq_of_row[t];
  const bool first = t == query_start[s];
  const int slot = state_slots[s];
  const float* kept = (first && positions[t] > 0 && slot >= 0) ? state + slot * state_stride + prev_off : nullptr;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    const float cur = ld(h + t * D + d);
    const float before = first ? (kept ? kept[d] : 0.0f) : ld(h + (t - 1) * D + d);
    const float diff = before - cur;
    for (int m = 0; m < n_mix; ++m) st(out + t * out_stride + static_cast<long long>(m) * D + d, fmaf(diff, mu[m * D + d], cur));
  }
}

template <typename T>
__global__ void __launch_bounds__(256) tanh_rows_kernel(const float* __restrict__ x, long long x_stride, T* __restrict__ out,
                                                        long long out_stride, int cols, long long total) {
  pdl_sync();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / cols;
  const int c = static_cast<int>(i % cols);
  st(out + t * out_stride + c, tanhf(x[t * x_stride + c]));
}

template <typename T>
__global__ void __launch_bounds__(256) time_mix_prep_kernel(const T* __restrict__ r, const T* __restrict__ k, const T* __restrict__ v,
                                                            long long in_stride, const float* __restrict__ w0, float* __restrict__ rn,
                                                            float* __restrict__ kn, float* __restrict__ vn, float* __restrict__ decay,
                                                            int n, long long total) {
  pdl_sync();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / n;
  const int c = static_cast<int>(i % n);
  rn[i] = ld(r + t * in_stride + c);
  kn[i] = ld(k + t * in_stride + c);
  vn[i] = ld(v + t * in_stride + c);
  decay[i] = expf(-expf(decay[i] + w0[c]));
}

template <typename T>
__global__ void __launch_bounds__(128) time_mix_out_kernel(const float* __restrict__ o, const T* __restrict__ gate, long long gate_stride,
                                                           const float* __restrict__ w, float eps, T* __restrict__ out, int heads,
                                                           int dim, long long items, const T* __restrict__ h, int D,
                                                           float* __restrict__ state, long long state_stride, long long prev_off,
                                                           const int* __restrict__ seq_of_row, const int* __restrict__ query_start,
                                                           const int* __restrict__ state_slots) {
  pdl_sync();
  const int lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= items) return;
  const long long t = item / heads;
  const int hd = static_cast<int>(item % heads);
  const float* x = o + item * dim;
  float ss = 0.0f;
  for (int d = lane; d < dim; d += 32) ss = fmaf(x[d], x[d], ss);
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(dim) + eps);
  for (int d = lane; d < dim; d += 32) {
    const float g = ld(gate + t * gate_stride + hd * dim + d);
    st(out + item * dim + d, ((x[d] * inv) * w[hd * dim + d]) * (g / (1.0f + expf(-g))));
  }
  // the heads of a sequence's last row share the copy of that row into the slot
  const int s = seq_of_row[t];
  const int slot = state_slots[s];
  if (slot >= 0 && t == query_start[s + 1] - 1) {
    float* kept = state + slot * state_stride + prev_off;
    for (int d = hd * 32 + lane; d < D; d += heads * 32) kept[d] = ld(h + t * D + d);
  }
}

}  // namespace tie

using namespace tie;

#define TIE_BY_DTYPE(dtype, CALL_F32, CALL_BF16) \
  do {                                           \
    if (dtype == TIE_F32) {                      \
      CALL_F32;                                  \
    } else if (dtype == TIE_BF16) {              \
      CALL_BF16;                                 \
    } else {                                     \
      set_error("unknown dtype code %d", dtype); \
      return kBadArgument;                       \
    }                                            \
  } while (0)

TIE_API int tie_token_shift_mix(int dtype, const void* h, const float* mu, int n_mix, const float* state, long long state_stride,
                                long long prev_off, const int* seq_of_row, const int* query_start, const int* positions,
                                const int* state_slots, void* out, long long out_stride, int tokens, int D, cudaStream_t s) {
  TIE_REQUIRE(tokens >= 0 && D > 0 && n_mix > 0 && out_stride >= static_cast<long long>(n_mix) * D, "token_shift_mix: bad sizes");
  if (tokens == 0) return kOk;
  TIE_BY_DTYPE(dtype,
               TIE_LAUNCH((token_shift_mix_kernel<float>), tokens, 256, 0, s, static_cast<const float*>(h), mu, n_mix, state, state_stride,
                          prev_off, seq_of_row, query_start, positions, state_slots, static_cast<float*>(out), out_stride, D),
               TIE_LAUNCH((token_shift_mix_kernel<__nv_bfloat16>), tokens, 256, 0, s, static_cast<const __nv_bfloat16*>(h), mu, n_mix, state,
                          state_stride, prev_off, seq_of_row, query_start, positions, state_slots, static_cast<__nv_bfloat16*>(out),
                          out_stride, D));
  TIE_RETURN_LAUNCH("token_shift_mix");
}

TIE_API int tie_tanh_rows(int dtype, const float* x, long long x_stride, void* out, long long out_stride, int tokens, int cols,
                          cudaStream_t s) {
  TIE_REQUIRE(tokens >= 0 && cols > 0, "tanh_rows: bad sizes");
  const long long total = static_cast<long long>(tokens) * cols;
  if (total == 0) return kOk;
  TIE_BY_DTYPE(dtype,
               TIE_LAUNCH((tanh_rows_kernel<float>), ceil_div(total, 256), 256, 0, s, x, x_stride, static_cast<float*>(out), out_stride, cols, total),
               TIE_LAUNCH((tanh_rows_kernel<__nv_bfloat16>), ceil_div(total, 256), 256, 0, s, x, x_stride, static_cast<__nv_bfloat16*>(out),
                          out_stride, cols, total));
  TIE_RETURN_LAUNCH("tanh_rows");
}

TIE_API int tie_time_mix_prep(int dtype, const void* r, const void* k, const void* v, long long in_stride, const float* w0, float* rn,
                              float* kn, float* vn, float* decay, int tokens, int n, cudaStream_t s) {
  TIE_REQUIRE(tokens >= 0 && n > 0, "time_mix_prep: bad sizes");
  const long long total = static_cast<long long>(tokens) * n;
  if (total == 0) return kOk;
  TIE_BY_DTYPE(dtype,
               TIE_LAUNCH((time_mix_prep_kernel<float>), ceil_div(total, 256), 256, 0, s, static_cast<const float*>(r), static_cast<const float*>(k),
                          static_cast<const float*>(v), in_stride, w0, rn, kn, vn, decay, n, total),
               TIE_LAUNCH((time_mix_prep_kernel<__nv_bfloat16>), ceil_div(total, 256), 256, 0, s, static_cast<const __nv_bfloat16*>(r),
                          static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v), in_stride, w0, rn, kn, vn, decay, n, total));
  TIE_RETURN_LAUNCH("time_mix_prep");
}

TIE_API int tie_time_mix_out(int dtype, const float* o, const void* gate, long long gate_stride, const float* w, float eps, void* out,
                             int tokens, int heads, int dim, const void* h, int D, float* state, long long state_stride,
                             long long prev_off, const int* seq_of_row, const int* query_start, const int* state_slots,
                             cudaStream_t s) {
  TIE_REQUIRE(tokens >= 0 && heads > 0 && dim > 0 && D > 0, "time_mix_out: bad sizes");
  const long long items = static_cast<long long>(tokens) * heads;
  if (items == 0) return kOk;
  TIE_BY_DTYPE(dtype,
               TIE_LAUNCH((time_mix_out_kernel<float>), ceil_div(items, 4), 128, 0, s, o, static_cast<const float*>(gate), gate_stride, w, eps,
                          static_cast<float*>(out), heads, dim, items, static_cast<const float*>(h), D, state, state_stride, prev_off,
                          seq_of_row, query_start, state_slots),
               TIE_LAUNCH((time_mix_out_kernel<__nv_bfloat16>), ceil_div(items, 4), 128, 0, s, o, static_cast<const __nv_bfloat16*>(gate),
                          gate_stride, w, eps, static_cast<__nv_bfloat16*>(out), heads, dim, items, static_cast<const __nv_bfloat16*>(h), D,
                          state, state_stride, prev_off, seq_of_row, query_start, state_slots));
  TIE_RETURN_LAUNCH("time_mix_out");
}
