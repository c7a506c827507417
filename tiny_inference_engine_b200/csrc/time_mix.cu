// What stands around the plain recurrence (delta_rule.cu, read-first mode) for a mixer that blends every input with
// the token before:
//
//   token_shift_concat  out[t] = [h[t] | h[t - 1]]; the row before the first row of a sequence's portion is the one its state
//                       slot keeps (zeros at position 0). A blend h + (h' - h) * mu times a weight W is [W (1 - mu) | W mu] times
//                       this row (the factors scale W's columns), so all blends' projections are one matrix product.
//   time_mix_prep       r, k, v (compute type) -> float rows; decay = exp(-exp(w2 tanh(inner) + w0)), float: the second step of
//                       the decay's projection runs here, over a few dozen inner channels
//   time_mix_out      (o / rms(o) per head) * w[h, :] * silu(gate) in the compute type; the sequence's last row of h
//                     becomes the row that its slot keeps
#include <math.h>

#include "common.cuh"

namespace tie {

template <typename T>
__global__ void __launch_bounds__(256) token_shift_concat_kernel(const T* __restrict__ h, const float* __restrict__ state,
                                                                 long long state_stride, long long prev_off,
                                                                 const int* __restrict__ seq_of_row, const int* __restrict__ query_start,
                                                                 const int* __restrict__ positions, const int* __restrict__ state_slots,
                                                                 T* __restrict__ out, int D) {
  pdl_sync();
  const long long t = blockIdx.x;
  const int s = seq_of_row[t];
  const bool first = t == query_start[s];
  const int slot = state_slots[s];
  const float* kept = (first && positions[t] > 0 && slot >= 0) ? state + slot * state_stride + prev_off : nullptr;
  T* row = out + t * 2 * D;
  for (int d = blockIdx.y * blockDim.x + threadIdx.x; d < D; d += gridDim.y * blockDim.x) {
    row[d] = h[t * D + d];
    if (first) st(row + D + d, kept ? kept[d] : 0.0f);
    else row[D + d] = h[(t - 1) * D + d];
  }
}

// Blocks of 256 decay channels of a token (a few tokens fill the GPU that way): tanh of the inner channels into shared memory,
// then a thread a decay channel.
template <typename T>
__global__ void __launch_bounds__(256) time_mix_prep_kernel(const T* __restrict__ proj, long long stride, int r_off, int k_off, int v_off,
                                                            int inner_off, int rank, const float* __restrict__ w2t,
                                                            const float* __restrict__ w0, float* __restrict__ rn, float* __restrict__ kn,
                                                            float* __restrict__ vn, float* __restrict__ decay, int n) {
  pdl_sync();
  extern __shared__ float inner[];
  const long long t = blockIdx.x;
  const T* row = proj + t * stride;
  for (int j = threadIdx.x; j < rank; j += blockDim.x) inner[j] = tanhf(ld(row + inner_off + j));
  __syncthreads();
  for (int c = blockIdx.y * blockDim.x + threadIdx.x; c < n; c += gridDim.y * blockDim.x) {
    rn[t * n + c] = ld(row + r_off + c);
    kn[t * n + c] = ld(row + k_off + c);
    vn[t * n + c] = ld(row + v_off + c);
    float z = 0.0f;
    for (int j = 0; j < rank; ++j) z = fmaf(w2t[static_cast<long long>(j) * n + c], inner[j], z);
    decay[t * n + c] = expf(-expf(z + w0[c]));
  }
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

TIE_API int tie_token_shift_concat(int dtype, const void* h, const float* state, long long state_stride, long long prev_off,
                                   const int* seq_of_row, const int* query_start, const int* positions, const int* state_slots,
                                   void* out, int tokens, int D, cudaStream_t s) {
  TIE_REQUIRE(tokens >= 0 && D > 0, "token_shift_concat: bad sizes");
  if (tokens == 0) return kOk;
  const int col_tiles = tokens >= 512 ? 1 : min(ceil_div(D, 256), 64);      // few rows: several blocks a row
  TIE_BY_DTYPE(dtype,
               TIE_LAUNCH((token_shift_concat_kernel<float>), dim3(tokens, col_tiles), 256, 0, s, static_cast<const float*>(h), state, state_stride, prev_off,
                          seq_of_row, query_start, positions, state_slots, static_cast<float*>(out), D),
               TIE_LAUNCH((token_shift_concat_kernel<__nv_bfloat16>), dim3(tokens, col_tiles), 256, 0, s, static_cast<const __nv_bfloat16*>(h), state,
                          state_stride, prev_off, seq_of_row, query_start, positions, state_slots, static_cast<__nv_bfloat16*>(out), D));
  TIE_RETURN_LAUNCH("token_shift_concat");
}

TIE_API int tie_time_mix_prep(int dtype, const void* proj, long long stride, int r_off, int k_off, int v_off, int inner_off, int rank,
                              const float* w2t, const float* w0, float* rn, float* kn, float* vn, float* decay, int tokens, int n,
                              cudaStream_t s) {
  TIE_REQUIRE(tokens >= 0 && n > 0 && rank > 0 && rank <= 8192, "time_mix_prep: bad sizes tokens=%d n=%d inner=%d", tokens, n, rank);
  if (tokens == 0) return kOk;
  const size_t smem = static_cast<size_t>(rank) * sizeof(float);
  const int col_tiles = tokens >= 512 ? 1 : min(ceil_div(n, 256), 64);
  TIE_BY_DTYPE(dtype,
               TIE_LAUNCH((time_mix_prep_kernel<float>), dim3(tokens, col_tiles), 256, smem, s, static_cast<const float*>(proj), stride, r_off, k_off, v_off,
                          inner_off, rank, w2t, w0, rn, kn, vn, decay, n),
               TIE_LAUNCH((time_mix_prep_kernel<__nv_bfloat16>), dim3(tokens, col_tiles), 256, smem, s, static_cast<const __nv_bfloat16*>(proj), stride, r_off,
                          k_off, v_off, inner_off, rank, w2t, w0, rn, kn, vn, decay, n));
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
