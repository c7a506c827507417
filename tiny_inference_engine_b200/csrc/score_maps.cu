// What stands around attention whose query heads read slices of wider key rows (attention_simt.cu, the `maps`
// launchers): the step between the stacked product and attention, and the two ways its float outputs become a
// layer's heads.
//
//   slice_norm_append   per token: every slice of `dim` of the q columns is divided by its root mean square and
//                       multiplied by a weight shared by all slices (in place; skipped without a weight), every slice
//                       of the k columns likewise on its way into the key plane, the v columns copied into the value
//                       plane. Key rows hold `k_row` elements per cached head, value rows `v_row`.
//   diff_combine        two maps a head, a [T, 2, H, vdim] (float, or the compute type): o = a1 - lambda a2,
//                       o / rms(o) * mult, times sigmoid(gate), into the compute type.
//   head_talk           a [T, H, G, vdim] (float, or the compute type; every head's weights on every kv head's values):
//                       out[t, h] = sum_g talk[h, g] a[t, g, kv head of h], into the compute type.
#include <math.h>

#include "common.cuh"

namespace tie {

template <typename T>
__global__ void __launch_bounds__(128) slice_norm_append_kernel(T* __restrict__ proj, long long stride, int q_off, int nq, int k_off,
                                                                int nk, int v_off, int v_width, int dim,
                                                                const float* __restrict__ wq, const float* __restrict__ wk, float eps,
                                                                const int* __restrict__ slots, T* __restrict__ k_cache,
                                                                T* __restrict__ v_cache, int kv_heads, int k_row, int v_row,
                                                                int page_size, int write_kv) {
  pdl_sync();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  const long long t = blockIdx.x;
  T* row = proj + t * stride;
  const int slot = write_kv ? slots[t] : -1;
  const long long page = slot >= 0 ? slot / page_size : 0, off = slot >= 0 ? slot % page_size : 0;
  const int slices = (wq ? nq : 0) + (slot >= 0 ? nk : 0);
  for (int i = blockIdx.y * warps + warp; i < slices; i += gridDim.y * warps) {
    const bool is_q = wq != nullptr && i < nq;
    const int j = is_q ? i : i - (wq ? nq : 0);
    T* src = row + (is_q ? q_off : k_off) + j * dim;
    const float* w = is_q ? wq : wk;
    float inv = 1.0f;
    if (w != nullptr) {
      float ss = 0.0f;
      for (int d = lane; d < dim; d += 32) {
        const float v = ld(src + d);
        ss = fmaf(v, v, ss);
      }
      ss = warp_sum(ss);
      inv = 1.0f / sqrtf(ss / static_cast<float>(dim) + eps);
    }
    T* dst = src;
    if (!is_q) {
      const int per_head = k_row / dim;      // slices a cached head holds
      const int c = j / per_head, sub = j % per_head;
      dst = k_cache + ((page * kv_heads + c) * page_size + off) * k_row + sub * dim;
    }
    for (int d = lane; d < dim; d += 32) {
      const float v = ld(src + d);
      st(dst + d, w != nullptr ? (v * inv) * w[d] : v);
    }
  }
  if (slot >= 0) {
    for (int j = blockIdx.y * blockDim.x + threadIdx.x; j < v_width; j += gridDim.y * blockDim.x) {
      const int c = j / v_row, d = j % v_row;
      v_cache[((page * kv_heads + c) * page_size + off) * v_row + d] = row[v_off + j];
    }
  }
}

template <typename T, typename A>
__global__ void __launch_bounds__(128) diff_combine_kernel(const A* __restrict__ a, const T* __restrict__ gate,
                                                           long long gate_stride, float lambda, float mult, float eps,
                                                           T* __restrict__ out, int heads, int vdim, long long items) {
  pdl_sync();
  const int lane = threadIdx.x & 31;
  const long long item = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= items) return;
  const long long t = item / heads;
  const int h = static_cast<int>(item % heads);
  const A* a1 = a + (t * 2 * heads + h) * vdim;
  const A* a2 = a1 + static_cast<long long>(heads) * vdim;
  float ss = 0.0f;
  for (int d = lane; d < vdim; d += 32) {
    const float o = ld(a1 + d) - lambda * ld(a2 + d);
    ss = fmaf(o, o, ss);
  }
  ss = warp_sum(ss);
  const float inv = 1.0f / sqrtf(ss / static_cast<float>(vdim) + eps);
  for (int d = lane; d < vdim; d += 32) {
    const float o = ld(a1 + d) - lambda * ld(a2 + d);
    float v = (o * inv) * mult;
    if (gate != nullptr) v *= 1.0f / (1.0f + expf(-ld(gate + t * gate_stride + h * vdim + d)));
    st(out + item * vdim + d, v);
  }
}

template <typename T, typename A>
__global__ void __launch_bounds__(256) head_talk_kernel(const A* __restrict__ a, const float* __restrict__ talk,
                                                        T* __restrict__ out, int heads, int kv_heads, int vdim) {
  pdl_sync();
  const long long t = blockIdx.x;
  const int per = heads / kv_heads;
  const A* row = a + t * heads * kv_heads * vdim;
  for (int i = threadIdx.x; i < heads * vdim; i += blockDim.x) {
    const int h = i / vdim, d = i % vdim;
    const int c = h / per;
    float acc = 0.0f;
    for (int g = 0; g < heads; ++g) acc = fmaf(talk[h * heads + g], ld(row + (g * kv_heads + c) * vdim + d), acc);
    st(out + t * heads * vdim + i, acc);
  }
}

}  // namespace tie

using namespace tie;

TIE_API int tie_slice_norm_append(int dtype, void* proj, long long stride, int q_off, int nq, int k_off, int nk, int v_off,
                                  int v_width, int dim, const float* wq, const float* wk, float eps, const int* slots,
                                  void* k_cache, void* v_cache, int tokens, int kv_heads, int k_row, int v_row, int page_size,
                                  int write_kv, cudaStream_t s) {
  TIE_REQUIRE(dim > 0 && nq >= 0 && nk >= 0 && tokens >= 0, "slice_norm_append: bad sizes");
  if (write_kv)
    TIE_REQUIRE(kv_heads > 0 && k_row > 0 && v_row > 0 && k_row % dim == 0 && nk * dim == kv_heads * k_row && v_width == kv_heads * v_row &&
                    page_size > 0 && slots && k_cache && v_cache,
                "slice_norm_append: %d key slices of %d and %d value columns do not fill %d cached heads of %d and %d", nk, dim,
                v_width, kv_heads, k_row, v_row);
  if (tokens == 0 || (!write_kv && wq == nullptr)) return kOk;
  const int slice_tiles = tokens >= 512 ? 1 : min(ceil_div((wq ? nq : 0) + (write_kv ? nk : 0), 4), 32);      // few rows: several blocks a row
  const dim3 grid(tokens, slice_tiles > 0 ? slice_tiles : 1);
  if (dtype == TIE_F32) {
    TIE_LAUNCH((slice_norm_append_kernel<float>), grid, 128, 0, s, static_cast<float*>(proj), stride, q_off, nq, k_off, nk, v_off,
               v_width, dim, wq, wk, eps, slots, static_cast<float*>(k_cache), static_cast<float*>(v_cache), kv_heads, k_row, v_row,
               page_size, write_kv);
  } else if (dtype == TIE_BF16) {
    TIE_LAUNCH((slice_norm_append_kernel<__nv_bfloat16>), grid, 128, 0, s, static_cast<__nv_bfloat16*>(proj), stride, q_off, nq,
               k_off, nk, v_off, v_width, dim, wq, wk, eps, slots, static_cast<__nv_bfloat16*>(k_cache),
               static_cast<__nv_bfloat16*>(v_cache), kv_heads, k_row, v_row, page_size, write_kv);
  } else {
    set_error("unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("slice_norm_append");
}

TIE_API int tie_diff_combine(int dtype, int a_f32, const void* a, const void* gate, long long gate_stride, float lambda, float mult,
                             float eps, void* out, int tokens, int heads, int vdim, cudaStream_t s) {
  TIE_REQUIRE(tokens >= 0 && heads > 0 && vdim > 0, "diff_combine: bad sizes tokens=%d heads=%d vdim=%d", tokens, heads, vdim);
  const long long items = static_cast<long long>(tokens) * heads;
  if (items == 0) return kOk;
  if (dtype == TIE_F32) {
    TIE_LAUNCH((diff_combine_kernel<float, float>), ceil_div(items, 4), 128, 0, s, static_cast<const float*>(a), static_cast<const float*>(gate),
               gate_stride, lambda, mult, eps, static_cast<float*>(out), heads, vdim, items);
  } else if (dtype == TIE_BF16 && a_f32) {
    TIE_LAUNCH((diff_combine_kernel<__nv_bfloat16, float>), ceil_div(items, 4), 128, 0, s, static_cast<const float*>(a),
               static_cast<const __nv_bfloat16*>(gate), gate_stride, lambda, mult, eps, static_cast<__nv_bfloat16*>(out), heads, vdim, items);
  } else if (dtype == TIE_BF16) {
    TIE_LAUNCH((diff_combine_kernel<__nv_bfloat16, __nv_bfloat16>), ceil_div(items, 4), 128, 0, s, static_cast<const __nv_bfloat16*>(a),
               static_cast<const __nv_bfloat16*>(gate), gate_stride, lambda, mult, eps, static_cast<__nv_bfloat16*>(out), heads, vdim, items);
  } else {
    set_error("unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("diff_combine");
}

TIE_API int tie_head_talk(int dtype, int a_f32, const void* a, const float* talk, void* out, int tokens, int heads, int kv_heads, int vdim,
                          cudaStream_t s) {
  TIE_REQUIRE(tokens >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && vdim > 0,
              "head_talk: bad sizes tokens=%d heads=%d/%d vdim=%d", tokens, heads, kv_heads, vdim);
  if (tokens == 0) return kOk;
  if (dtype == TIE_F32) {
    TIE_LAUNCH((head_talk_kernel<float, float>), tokens, 256, 0, s, static_cast<const float*>(a), talk, static_cast<float*>(out), heads, kv_heads, vdim);
  } else if (dtype == TIE_BF16 && a_f32) {
    TIE_LAUNCH((head_talk_kernel<__nv_bfloat16, float>), tokens, 256, 0, s, static_cast<const float*>(a), talk, static_cast<__nv_bfloat16*>(out),
               heads, kv_heads, vdim);
  } else if (dtype == TIE_BF16) {
    TIE_LAUNCH((head_talk_kernel<__nv_bfloat16, __nv_bfloat16>), tokens, 256, 0, s, static_cast<const __nv_bfloat16*>(a), talk,
               static_cast<__nv_bfloat16*>(out), heads, kv_heads, vdim);
  } else {
    set_error("unknown dtype code %d", dtype);
    return kBadArgument;
  }
  TIE_RETURN_LAUNCH("head_talk");
}
