// A norm without statistics, and a position added to the embedding.
//
//   add_tanh_norm   x += sa * A + sb * B (float, in place; each of A, B a tensor in the compute type or the float
//                   partial sums of a split product, added in split order; either may be absent), then
//                   out = tanh(alpha * x) * w + b in the compute type. With `rows`, out[i] comes from row rows[i]
//                   and x is left as it is.
//   sinusoid_add    x[t, 2i] += sin(p / base^(2i/D)), x[t, 2i + 1] += cos of the same angle, p the row's position.
//                   The angle is formed in double precision, so that it is the same number at position 5 and 5,000.
#include <math.h>

#include "common.cuh"

namespace tie {

struct Term {
  const void* tensor;       // [T, D] in the compute type, or null
  const float* partial;     // [splits, T, D] float, or null
  long long stride;         // T * D
  int splits;
  float scale;
};

template <typename T>
__device__ __forceinline__ float term_at(const Term& term, long long at) {
  float v = 0.0f;
  if (term.tensor != nullptr) v = ld(static_cast<const T*>(term.tensor) + at);
  else if (term.partial != nullptr) {
    for (int z = 0; z < term.splits; ++z) v += term.partial[z * term.stride + at];
  } else return 0.0f;
  return term.scale * v;
}

template <typename T>
__global__ void __launch_bounds__(256) add_tanh_norm_kernel(float* __restrict__ x, Term a, Term b, const int* __restrict__ rows,
                                                            float alpha, const float* __restrict__ w, const float* __restrict__ bias,
                                                            T* __restrict__ out, int n, int D) {
  pdl_sync();
  const long long total = static_cast<long long>(n) * D;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int d = static_cast<int>(i % D);
    const long long r = rows ? rows[i / D] : i / D;
    const long long at = r * D + d;
    // a first, then b: the order of the sum is a fixed one
    float v = x[at];
    v += term_at<T>(a, at);
    v += term_at<T>(b, at);
    if (rows == nullptr && (a.tensor || a.partial || b.tensor || b.partial)) x[at] = v;
    st(out + i, fmaf(tanhf(alpha * v), w[d], bias[d]));
  }
}

// Four columns a thread (D a multiple of four, every pointer on a 16-byte boundary; the terms' rows likewise).
template <typename T>
__device__ __forceinline__ void term_add4(const Term& term, long long at, float (&v)[4]) {
  if (term.tensor != nullptr) {
    float d[4];
    load4(static_cast<const T*>(term.tensor) + at, d);
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = fmaf(term.scale, d[e], v[e]);
  } else if (term.partial != nullptr) {
    float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for (int z = 0; z < term.splits; ++z) {
      float d[4];
      load4(term.partial + z * term.stride + at, d);
#pragma unroll
      for (int e = 0; e < 4; ++e) sum[e] += d[e];
    }
#pragma unroll
    for (int e = 0; e < 4; ++e) v[e] = fmaf(term.scale, sum[e], v[e]);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) add_tanh_norm_vec4_kernel(float* __restrict__ x, Term a, Term b, const int* __restrict__ rows,
                                                                 float alpha, const float* __restrict__ w, const float* __restrict__ bias,
                                                                 T* __restrict__ out, int n, int D) {
  pdl_sync();
  const int quads = D / 4;
  const long long total = static_cast<long long>(n) * quads;
  const bool adds = a.tensor || a.partial || b.tensor || b.partial;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int d = static_cast<int>(i % quads) * 4;
    const long long r = rows ? rows[i / quads] : i / quads;
    const long long at = r * D + d;
    float v[4], ww[4], bb[4], o[4];
    load4(x + at, v);
    term_add4<T>(a, at, v);
    term_add4<T>(b, at, v);
    if (rows == nullptr && adds) store4(x + at, v);
    load4(w + d, ww);
    load4(bias + d, bb);
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] = fmaf(tanhf(alpha * v[e]), ww[e], bb[e]);
    store4(out + (i / quads) * D + d, o);
  }
}

__global__ void __launch_bounds__(256) sinusoid_add_kernel(float* __restrict__ x, const int* __restrict__ positions, int T,
                                                           int D, double log_base) {
  pdl_sync();
  const int pairs = (D + 1) / 2;
  const long long total = static_cast<long long>(T) * pairs;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int p = static_cast<int>(i % pairs);
    const long long t = i / pairs;
    const double angle = static_cast<double>(positions[t]) * exp(-2.0 * p / D * log_base);
    double sn, cs;
    sincos(angle, &sn, &cs);
    x[t * D + 2 * p] += static_cast<float>(sn);
    if (2 * p + 1 < D) x[t * D + 2 * p + 1] += static_cast<float>(cs);
  }
}

}  // namespace tie

using namespace tie;

TIE_API int tie_add_tanh_norm(int dtype, float* x, const void* a, const float* a_part, long long a_stride, int a_splits,
                              float a_scale, const void* b, const float* b_part, long long b_stride, int b_splits, float b_scale,
                              const int* rows, float alpha, const float* w, const float* bias, void* out, int n, int D,
                              cudaStream_t s) {
  TIE_REQUIRE(n >= 0 && D > 0, "add_tanh_norm: bad sizes n=%d D=%d", n, D);
  if (n == 0) return kOk;
  const Term ta{a, a_part, a_stride, a_splits, a_scale}, tb{b, b_part, b_stride, b_splits, b_scale};
  const int blocks = static_cast<int>(min(static_cast<long long>(148 * 8), (static_cast<long long>(n) * D + 255) / 256));
  auto on16 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool vec4 = D % 4 == 0 && on16(x) && on16(a) && on16(a_part) && on16(b) && on16(b_part) && on16(w) && on16(bias) && on16(out) &&
                    a_stride % 4 == 0 && b_stride % 4 == 0;
  const int blocks4 = static_cast<int>(min(static_cast<long long>(148 * 8), (static_cast<long long>(n) * (D / 4) + 255) / 256));
  if (dtype == TIE_F32) {
    if (vec4) TIE_LAUNCH((add_tanh_norm_vec4_kernel<float>), blocks4, 256, 0, s, x, ta, tb, rows, alpha, w, bias, static_cast<float*>(out), n, D);
    else TIE_LAUNCH((add_tanh_norm_kernel<float>), blocks, 256, 0, s, x, ta, tb, rows, alpha, w, bias, static_cast<float*>(out), n, D);
  } else if (dtype == TIE_BF16) {
    if (vec4)
      TIE_LAUNCH((add_tanh_norm_vec4_kernel<__nv_bfloat16>), blocks4, 256, 0, s, x, ta, tb, rows, alpha, w, bias,
                 static_cast<__nv_bfloat16*>(out), n, D);
    else
      TIE_LAUNCH((add_tanh_norm_kernel<__nv_bfloat16>), blocks, 256, 0, s, x, ta, tb, rows, alpha, w, bias,
                 static_cast<__nv_bfloat16*>(out), n, D);
  } else {
    set_error("unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("add_tanh_norm");
}

TIE_API int tie_sinusoid_add(float* x, const int* positions, int T, int D, float base, cudaStream_t s) {
  TIE_REQUIRE(T >= 0 && D > 0 && base > 0.0f, "sinusoid_add: bad sizes T=%d D=%d base=%g", T, D, static_cast<double>(base));
  if (T == 0) return kOk;
  const long long total = static_cast<long long>(T) * ((D + 1) / 2);
  const int blocks = static_cast<int>(min(static_cast<long long>(148 * 8), (total + 255) / 256));
  TIE_LAUNCH(sinusoid_add_kernel, blocks, 256, 0, s, x, positions, T, D, log(static_cast<double>(base)));
  TIE_RETURN_LAUNCH("sinusoid_add");
}
