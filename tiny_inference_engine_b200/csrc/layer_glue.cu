// Small kernels between the matrix products of layers that norm a sublayer's output before adding it:
//
//   add_normed_rmsnorm  x += mult * ((y * inv(y)) * wb),  y = delta (+ bias);  out = (x * inv(x)) * w
//                       the residual add of a sublayer whose output passes a norm of its own first, fused with
//                       the norm ahead of the next sublayer. All of it in float: y, both sums, the residual.
//   glu_clamped         out = g' * sigmoid(slope * g') * (u' + up_shift),  g' = min(g, limit), u' = clamp(u, +-limit)
//   sigmoid_gate_mul    y *= sigmoid(gate)  (a gate on the heads' outputs)
//   scale_rows          x *= c  (float rows: the logits of a model that scales them)
#include <math.h>

#include "common.cuh"

namespace tie {

// One block per output row. The row is kept in shared memory between the passes (dim floats).
template <typename T>
__global__ void __launch_bounds__(1024) add_normed_rmsnorm_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                                                 const float* __restrict__ part, long long part_stride,
                                                                 int splits, const float* __restrict__ bias,
                                                                 const float* __restrict__ wb, float eps_b, float mult,
                                                                 const int* __restrict__ rows, const float* __restrict__ w,
                                                                 float eps, T* __restrict__ out, int dim) {
  pdl_sync();
  extern __shared__ float row[];
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[t] : t) * dim;
  float* xr = x + src;
  const T* dr = delta ? delta + src : nullptr;
  const float* pr = part ? part + src : nullptr;
  float ss = 0.0f;
  const int nt = blockDim.x;
  for (int k0 = threadIdx.x; k0 < dim; k0 += 4 * nt) {     // four elements a thread at a time, their loads in flight together
    float y[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (dr) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        if (k0 + i * nt < dim) y[i] = ld(dr + k0 + i * nt);
    } else {                                                // split by split: each element still adds in split order
#pragma unroll 4
      for (int z = 0; z < splits; ++z) {
        const float* pz = pr + static_cast<long long>(z) * part_stride;
#pragma unroll
        for (int i = 0; i < 4; ++i)
          if (k0 + i * nt < dim) y[i] += pz[k0 + i * nt];
      }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + i * nt;
      if (k < dim) {
        if (bias) y[i] += bias[k];
        row[k] = y[i];
        ss += y[i] * y[i];
      }
    }
  }
  ss = block_sum(ss, scratch);
  const float inv_y = 1.0f / sqrtf(ss / static_cast<float>(dim) + eps_b);
  float sx = 0.0f;
  for (int k = threadIdx.x; k < dim; k += blockDim.x) {
    const float v = xr[k] + mult * ((row[k] * inv_y) * wb[k]);
    if (rows == nullptr) xr[k] = v;
    row[k] = v;
    sx += v * v;
  }
  sx = block_sum(sx, scratch);
  const float inv_x = 1.0f / sqrtf(sx / static_cast<float>(dim) + eps);
  T* o = out + static_cast<size_t>(t) * dim;
  for (int k = threadIdx.x; k < dim; k += blockDim.x) st(o + k, (row[k] * inv_x) * w[k]);
}

// The same for rows of whole 16-byte pieces (dim % 4 == 0): every access is four elements wide.
template <typename T>
__global__ void __launch_bounds__(1024) add_normed_rmsnorm_vec4_kernel(float* __restrict__ x, const T* __restrict__ delta,
                                                                      const float* __restrict__ part, long long part_stride,
                                                                      int splits, const float* __restrict__ bias,
                                                                      const float* __restrict__ wb, float eps_b, float mult,
                                                                      const int* __restrict__ rows, const float* __restrict__ w,
                                                                      float eps, T* __restrict__ out, int dim) {
  pdl_sync();
  extern __shared__ float row[];
  __shared__ float scratch[33];
  const int t = blockIdx.x;
  const size_t src = static_cast<size_t>(rows ? rows[t] : t) * dim;
  float* xr = x + src;
  const T* dr = delta ? delta + src : nullptr;
  const float* pr = part ? part + src : nullptr;
  float ss = 0.0f;
  for (int k = 4 * threadIdx.x; k < dim; k += 4 * blockDim.x) {
    float y[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    if (dr) {
      load4(dr + k, y);
    } else {                                                // split by split: each element adds in split order
#pragma unroll 4
      for (int z = 0; z < splits; ++z) {
        float p[4];
        load4(pr + static_cast<long long>(z) * part_stride + k, p);
#pragma unroll
        for (int i = 0; i < 4; ++i) y[i] += p[i];
      }
    }
    if (bias) {
      float b[4];
      load4(bias + k, b);
#pragma unroll
      for (int i = 0; i < 4; ++i) y[i] += b[i];
    }
    store4(row + k, y);
#pragma unroll
    for (int i = 0; i < 4; ++i) ss += y[i] * y[i];
  }
  ss = block_sum(ss, scratch);
  const float inv_y = 1.0f / sqrtf(ss / static_cast<float>(dim) + eps_b);
  float sx = 0.0f;
  for (int k = 4 * threadIdx.x; k < dim; k += 4 * blockDim.x) {      // each thread its own elements of `row`
    float xv[4], y[4], g[4];
    load4(xr + k, xv);
    load4(row + k, y);
    load4(wb + k, g);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      xv[i] = xv[i] + mult * ((y[i] * inv_y) * g[i]);
      sx += xv[i] * xv[i];
    }
    if (rows == nullptr) store4(xr + k, xv);
    store4(row + k, xv);
  }
  sx = block_sum(sx, scratch);
  const float inv_x = 1.0f / sqrtf(sx / static_cast<float>(dim) + eps);
  T* o = out + static_cast<size_t>(t) * dim;
  for (int k = 4 * threadIdx.x; k < dim; k += 4 * blockDim.x) {
    float v[4], g[4];
    load4(row + k, v);
    load4(w + k, g);
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = (v[i] * inv_x) * g[i];
    store4(o + k, v);
  }
}

template <typename T>
__global__ void glu_clamped_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, long long total, float limit,
                                   float slope, float up_shift) {
  pdl_sync();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / inter;
  const int c = static_cast<int>(i % inter);
  const float g = fminf(ld(gu + t * 2 * inter + c), limit);
  const float u = fminf(fmaxf(ld(gu + t * 2 * inter + inter + c), -limit), limit);
  st(out + i, (g / (1.0f + expf(-slope * g))) * (u + up_shift));
}

// One hidden layer's activation in two branches that meet at zero with the slope 1/2:
//   z > 0: c_pos z^2 + z / 2;   z <= 0: c_neg (exp(z) - 1 - z) + z / 2.
__device__ __forceinline__ float two_branch(float v, float c_pos, float c_neg) {
  return v > 0.0f ? fmaf(c_pos * v, v, 0.5f * v) : fmaf(c_neg, expm1f(v) - v, 0.5f * v);
}

template <typename T>
__global__ void two_branch_unit_kernel(const T* __restrict__ z, T* __restrict__ out, long long total, float c_pos, float c_neg) {
  pdl_sync();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  st(out + i, two_branch(ld(z + i), c_pos, c_neg));
}

// 16 bytes a thread.
template <typename T>
__global__ void two_branch_unit_vec_kernel(const T* __restrict__ z, T* __restrict__ out, long long pieces, float c_pos, float c_neg) {
  pdl_sync();
  constexpr int V = Vec16<T>::N;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= pieces) return;
  Vec16<T> v;
  v.load(z + i * V);
#pragma unroll
  for (int e = 0; e < V; ++e) v.v[e] = two_branch(v.v[e], c_pos, c_neg);
  v.store(out + i * V);
}

template <typename T>
__global__ void sigmoid_gate_mul_kernel(T* __restrict__ y, long long y_stride, const T* __restrict__ gate,
                                        long long gate_stride, int width, long long total) {
  pdl_sync();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / width;
  const int c = static_cast<int>(i % width);
  const float g = ld(gate + t * gate_stride + c);
  T* p = y + t * y_stride + c;
  st(p, ld(p) / (1.0f + expf(-g)));
}

// The same two, 16 bytes a thread (rows whose widths and strides are whole 16-byte pieces).
template <typename T>
__global__ void glu_clamped_vec_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter, long long total_vecs, float limit,
                                       float slope, float up_shift) {
  pdl_sync();
  constexpr int V = Vec16<T>::N;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total_vecs) return;
  const int per_row = inter / V;
  const long long t = i / per_row;
  const int c = static_cast<int>(i % per_row) * V;
  Vec16<T> g, u, y;
  g.load(gu + t * 2 * inter + c);
  u.load(gu + t * 2 * inter + inter + c);
#pragma unroll
  for (int e = 0; e < V; ++e) {
    const float gv = fminf(g.v[e], limit);
    const float uv = fminf(fmaxf(u.v[e], -limit), limit);
    y.v[e] = (gv / (1.0f + expf(-slope * gv))) * (uv + up_shift);
  }
  y.store(out + t * inter + c);
}

template <typename T>
__global__ void sigmoid_gate_mul_vec_kernel(T* __restrict__ y, long long y_stride, const T* __restrict__ gate,
                                            long long gate_stride, int width, long long total_vecs) {
  pdl_sync();
  constexpr int V = Vec16<T>::N;
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total_vecs) return;
  const int per_row = width / V;
  const long long t = i / per_row;
  const int c = static_cast<int>(i % per_row) * V;
  Vec16<T> a, g;
  a.load(y + t * y_stride + c);
  g.load(gate + t * gate_stride + c);
#pragma unroll
  for (int e = 0; e < V; ++e) a.v[e] = a.v[e] / (1.0f + expf(-g.v[e]));
  a.store(y + t * y_stride + c);
}

__global__ void scale_rows_kernel(float* __restrict__ x, long long stride, int width, long long total, float c) {
  pdl_sync();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  x[(i / width) * stride + i % width] *= c;
}

template <typename T>
int launch_add_normed_rmsnorm(float* x, const void* delta, const float* part, long long part_stride, int splits,
                              const float* bias, const float* wb, float eps_b, float mult, const int* rows,
                              const float* w, float eps, void* out, int n, int dim, cudaStream_t s) {
  if (n == 0) return kOk;
  const size_t smem = static_cast<size_t>(dim) * sizeof(float);
  auto kernel = add_normed_rmsnorm_kernel<T>;
  if (smem > 48 * 1024) {
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) {
      set_error("add_normed_rmsnorm: rows of %d floats do not fit shared memory", dim);
      return kBadArgument;
    }
  }
  const auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  if (dim % 4 == 0 && part_stride % 4 == 0 && aligned(x) && aligned(delta) && aligned(part) && aligned(bias) && aligned(wb) &&
      aligned(w) && aligned(out)) {
    auto vec = add_normed_rmsnorm_vec4_kernel<T>;
    if (smem > 48 * 1024) cudaFuncSetAttribute(vec, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    TIE_LAUNCH(vec, n, dim >= 8192 ? 1024 : (dim >= 2048 ? 512 : (dim >= 1024 ? 256 : 128)), smem, s, x, static_cast<const T*>(delta),
               part, part_stride, splits, bias, wb, eps_b, mult, rows, w, eps, static_cast<T*>(out), dim);
    TIE_RETURN_LAUNCH("add_normed_rmsnorm");
  }
  TIE_LAUNCH(kernel, n, dim >= 4096 ? 1024 : (dim >= 2048 ? 512 : (dim >= 512 ? 256 : 128)), smem, s, x, static_cast<const T*>(delta), part, part_stride, splits, bias, wb,
             eps_b, mult, rows, w, eps, static_cast<T*>(out), dim);
  TIE_RETURN_LAUNCH("add_normed_rmsnorm");
}

}  // namespace tie

using namespace tie;

TIE_API int tie_add_normed_rmsnorm(int dtype, float* x, const void* delta, const float* part, long long part_stride,
                                   int splits, const float* bias, const float* wb, float eps_b, float mult,
                                   const int* rows, const float* w, float eps, void* out, int n, int dim, cudaStream_t s) {
  TIE_REQUIRE(n >= 0 && dim > 0 && dim <= 56 * 1024 && (delta != nullptr || (part != nullptr && splits > 0)),
              "add_normed_rmsnorm: bad sizes n=%d dim=%d, or nothing to add", n, dim);
  if (dtype == TIE_F32)
    return launch_add_normed_rmsnorm<float>(x, delta, part, part_stride, splits, bias, wb, eps_b, mult, rows, w, eps, out, n, dim, s);
  if (dtype == TIE_BF16)
    return launch_add_normed_rmsnorm<__nv_bfloat16>(x, delta, part, part_stride, splits, bias, wb, eps_b, mult, rows, w, eps, out, n,
                                                    dim, s);
  set_error("unknown dtype code %d", dtype);
  return kBadArgument;
}

TIE_API int tie_glu_clamped(int dtype, const void* gu, void* out, int tokens, int inter, float limit, float slope,
                            float up_shift, cudaStream_t s) {
  TIE_REQUIRE(tokens >= 0 && inter > 0, "glu_clamped: bad sizes tokens=%d inter=%d", tokens, inter);
  const long long total = static_cast<long long>(tokens) * inter;
  if (total == 0) return kOk;
  const bool aligned = reinterpret_cast<uintptr_t>(gu) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
  if (dtype == TIE_F32) {
    if (aligned && inter % 4 == 0)
      TIE_LAUNCH((glu_clamped_vec_kernel<float>), ceil_div(total / 4, 256), 256, 0, s, static_cast<const float*>(gu),
                 static_cast<float*>(out), inter, total / 4, limit, slope, up_shift);
    else
      TIE_LAUNCH((glu_clamped_kernel<float>), ceil_div(total, 256), 256, 0, s, static_cast<const float*>(gu), static_cast<float*>(out),
                 inter, total, limit, slope, up_shift);
  } else if (dtype == TIE_BF16) {
    if (aligned && inter % 8 == 0)
      TIE_LAUNCH((glu_clamped_vec_kernel<__nv_bfloat16>), ceil_div(total / 8, 256), 256, 0, s, static_cast<const __nv_bfloat16*>(gu),
                 static_cast<__nv_bfloat16*>(out), inter, total / 8, limit, slope, up_shift);
    else
      TIE_LAUNCH((glu_clamped_kernel<__nv_bfloat16>), ceil_div(total, 256), 256, 0, s, static_cast<const __nv_bfloat16*>(gu),
                 static_cast<__nv_bfloat16*>(out), inter, total, limit, slope, up_shift);
  } else {
    set_error("unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("glu_clamped");
}

TIE_API int tie_two_branch_unit(int dtype, const void* z, void* out, long long total, float c_pos, float c_neg, cudaStream_t s) {
  TIE_REQUIRE(total >= 0, "two_branch_unit: bad size");
  if (total == 0) return kOk;
  const bool aligned = reinterpret_cast<uintptr_t>(z) % 16 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
  if (dtype == TIE_F32) {
    if (aligned && total % 4 == 0)
      TIE_LAUNCH((two_branch_unit_vec_kernel<float>), ceil_div(total / 4, 256), 256, 0, s, static_cast<const float*>(z), static_cast<float*>(out),
                 total / 4, c_pos, c_neg);
    else
      TIE_LAUNCH((two_branch_unit_kernel<float>), ceil_div(total, 256), 256, 0, s, static_cast<const float*>(z), static_cast<float*>(out), total,
                 c_pos, c_neg);
  } else if (dtype == TIE_BF16) {
    if (aligned && total % 8 == 0)
      TIE_LAUNCH((two_branch_unit_vec_kernel<__nv_bfloat16>), ceil_div(total / 8, 256), 256, 0, s, static_cast<const __nv_bfloat16*>(z),
                 static_cast<__nv_bfloat16*>(out), total / 8, c_pos, c_neg);
    else
      TIE_LAUNCH((two_branch_unit_kernel<__nv_bfloat16>), ceil_div(total, 256), 256, 0, s, static_cast<const __nv_bfloat16*>(z),
                 static_cast<__nv_bfloat16*>(out), total, c_pos, c_neg);
  } else {
    set_error("unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("two_branch_unit");
}

TIE_API int tie_sigmoid_gate_mul(int dtype, void* y, long long y_stride, const void* gate, long long gate_stride, int tokens,
                                 int width, cudaStream_t s) {
  TIE_REQUIRE(tokens >= 0 && width > 0, "sigmoid_gate_mul: bad sizes tokens=%d width=%d", tokens, width);
  const long long total = static_cast<long long>(tokens) * width;
  if (total == 0) return kOk;
  const int vec = dtype == TIE_F32 ? 4 : 8;
  const bool aligned = reinterpret_cast<uintptr_t>(y) % 16 == 0 && reinterpret_cast<uintptr_t>(gate) % 16 == 0 &&
                       width % vec == 0 && y_stride % vec == 0 && gate_stride % vec == 0;
  if (dtype == TIE_F32) {
    if (aligned)
      TIE_LAUNCH((sigmoid_gate_mul_vec_kernel<float>), ceil_div(total / 4, 256), 256, 0, s, static_cast<float*>(y), y_stride,
                 static_cast<const float*>(gate), gate_stride, width, total / 4);
    else
      TIE_LAUNCH((sigmoid_gate_mul_kernel<float>), ceil_div(total, 256), 256, 0, s, static_cast<float*>(y), y_stride,
                 static_cast<const float*>(gate), gate_stride, width, total);
  } else if (dtype == TIE_BF16) {
    if (aligned)
      TIE_LAUNCH((sigmoid_gate_mul_vec_kernel<__nv_bfloat16>), ceil_div(total / 8, 256), 256, 0, s, static_cast<__nv_bfloat16*>(y),
                 y_stride, static_cast<const __nv_bfloat16*>(gate), gate_stride, width, total / 8);
    else
      TIE_LAUNCH((sigmoid_gate_mul_kernel<__nv_bfloat16>), ceil_div(total, 256), 256, 0, s, static_cast<__nv_bfloat16*>(y), y_stride,
                 static_cast<const __nv_bfloat16*>(gate), gate_stride, width, total);
  } else {
    set_error("unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("sigmoid_gate_mul");
}

TIE_API int tie_scale_rows(float* x, long long stride, int rows, int width, float c, cudaStream_t s) {
  TIE_REQUIRE(rows >= 0 && width > 0, "scale_rows: bad sizes rows=%d width=%d", rows, width);
  const long long total = static_cast<long long>(rows) * width;
  if (total == 0) return kOk;
  TIE_LAUNCH(scale_rows_kernel, ceil_div(total, 256), 256, 0, s, x, stride, width, total, c);
  TIE_RETURN_LAUNCH("scale_rows");
}
