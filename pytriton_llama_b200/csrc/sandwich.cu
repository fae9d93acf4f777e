// The norm after a sub-layer, the residual sum, the weighted sum over the results of all layers so far and
// the norm before the next sub-layer, one block per token row, float32 throughout:
//
//   u = a0                                                   (members == 0)
//   u = (1 / members) * sum_m a_m * rsqrt(mean(a_m^2) + eps) * w_m     (members 1 or 2: the mean of normed outputs)
//   post == nullptr:  y = u, nothing else                    (the mean alone)
//   X = residual + u * rsqrt(mean(u^2) + eps) * post
//   results given:    results[index][row] = X;   s = sum_{j < index} c[j] * results[j][row] + c[index] * X
//   else              s = X
//   residual <- s                                            (the stream, in place)
//   next given:       y = s * rsqrt(mean(s^2) + eps) * next  (element type T)
//
// Rows of up to 4,096 entries in whole packets take the fast form: a thread holds its share of the row (up to 16
// entries) in registers, requests everything it reads from memory -- the sub-layer outputs, the residual, the earlier
// results -- before the first sum over the block, and only then waits; the general form walks the row once per step.
//
// A is the element type of the sub-layer outputs (the compute type, or float32 from a routed feed-forward).
// The row is held in shared memory between the walks; with rows of whole 16-byte packets every walk moves
// packets.  Sums run over a thread's elements in ascending order and over the threads in a fixed tree, so a
// row's result does not depend on what else the step holds.
#include "common.cuh"

namespace ptl {

template <typename A>
__device__ __forceinline__ float sw_sumsq(const A* __restrict__ a, int width, bool vec, float* red) {
  float s = 0.f;
  if (vec) {
    constexpr int VN = Vec16<A>::N;
    for (int i = threadIdx.x * VN; i < width; i += blockDim.x * VN) {
      const Vec16<A> v = load16(a + i);
#pragma unroll
      for (int e = 0; e < VN; ++e) s = fmaf(v.get(e), v.get(e), s);
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) { const float v = to_f32(a[i]); s = fmaf(v, v, s); }
  }
  return block_sum(s, red);
}

template <typename T, typename A>
__global__ void __launch_bounds__(256)
post_norm_add_kernel(const A* __restrict__ a0, const A* __restrict__ a1, const float* __restrict__ w0,
                     const float* __restrict__ w1, int members, const float* __restrict__ post, float eps,
                     float* __restrict__ residual, float* __restrict__ results, long long result_stride, int index,
                     const float* __restrict__ coeffs, const float* __restrict__ next, T* __restrict__ y, int width, int vec) {
  extern __shared__ __align__(16) float sw_row[];
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();
  const size_t row = (size_t)blockIdx.x * width;
  a0 += row;
  if (a1) a1 += row;
  const float inv_w = 1.0f / (float)width;
  // u into shared memory
  if (members > 0) {
    const float r0 = 1.0f / sqrtf(sw_sumsq(a0, width, vec, red) * inv_w + eps);
    const float r1 = members > 1 ? 1.0f / sqrtf(sw_sumsq(a1, width, vec, red) * inv_w + eps) : 0.f;
    const float share = 1.0f / (float)members;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      float u = to_f32(a0[i]) * r0 * w0[i];
      if (members > 1) u += to_f32(a1[i]) * r1 * w1[i];
      sw_row[i] = u * share;
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) sw_row[i] = to_f32(a0[i]);
  }
  if (!post) {
    __syncthreads();
    for (int i = threadIdx.x; i < width; i += blockDim.x) y[row + i] = from_f32<T>(sw_row[i]);
    return;
  }
  float sq = 0.f;
  for (int i = threadIdx.x; i < width; i += blockDim.x) sq = fmaf(sw_row[i], sw_row[i], sq);     // a thread's own elements
  const float ru = 1.0f / sqrtf(block_sum(sq, red) * inv_w + eps);
  float* res = residual + row;
  float* mine = results ? results + (size_t)index * result_stride + row : nullptr;
  sq = 0.f;
  if (vec) {
    for (int i = threadIdx.x * 4; i < width; i += blockDim.x * 4) {
      const float4 r4 = *reinterpret_cast<const float4*>(res + i);
      const float4 p4 = *reinterpret_cast<const float4*>(post + i);
      const float4 u4 = *reinterpret_cast<const float4*>(sw_row + i);
      float4 x = make_float4(fmaf(u4.x * ru, p4.x, r4.x), fmaf(u4.y * ru, p4.y, r4.y), fmaf(u4.z * ru, p4.z, r4.z),
                             fmaf(u4.w * ru, p4.w, r4.w));
      if (mine) {
        *reinterpret_cast<float4*>(mine + i) = x;
        const float c = coeffs[index];
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        const float* base = results + row + i;
        int j = 0;
        for (; j + 4 <= index; j += 4) {      // four earlier results requested together, added in ascending order
          float4 h[4];
#pragma unroll
          for (int u = 0; u < 4; ++u) h[u] = *reinterpret_cast<const float4*>(base + (size_t)(j + u) * result_stride);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float cj = coeffs[j + u];
            s.x = fmaf(cj, h[u].x, s.x); s.y = fmaf(cj, h[u].y, s.y); s.z = fmaf(cj, h[u].z, s.z); s.w = fmaf(cj, h[u].w, s.w);
          }
        }
        for (; j < index; ++j) {
          const float cj = coeffs[j];
          const float4 h = *reinterpret_cast<const float4*>(base + (size_t)j * result_stride);
          s.x = fmaf(cj, h.x, s.x); s.y = fmaf(cj, h.y, s.y); s.z = fmaf(cj, h.z, s.z); s.w = fmaf(cj, h.w, s.w);
        }
        x = make_float4(fmaf(c, x.x, s.x), fmaf(c, x.y, s.y), fmaf(c, x.z, s.z), fmaf(c, x.w, s.w));
      }
      *reinterpret_cast<float4*>(res + i) = x;
      *reinterpret_cast<float4*>(sw_row + i) = x;
      sq = fmaf(x.x, x.x, sq); sq = fmaf(x.y, x.y, sq); sq = fmaf(x.z, x.z, sq); sq = fmaf(x.w, x.w, sq);
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
      float x = fmaf(sw_row[i] * ru, post[i], res[i]);
      if (mine) {
        mine[i] = x;
        float s = 0.f;
        for (int j = 0; j < index; ++j) s = fmaf(coeffs[j], results[(size_t)j * result_stride + row + i], s);
        x = fmaf(coeffs[index], x, s);
      }
      res[i] = x;
      sw_row[i] = x;
      sq = fmaf(x, x, sq);
    }
  }
  if (!next) return;
  const float rs = 1.0f / sqrtf(block_sum(sq, red) * inv_w + eps);
  if (vec) {
    constexpr int VN = Vec16<T>::N;
    for (int i = threadIdx.x * VN; i < width; i += blockDim.x * VN) {
      Vec16<T> v;
#pragma unroll
      for (int e = 0; e < VN; ++e) v.set(e, sw_row[i + e] * rs * next[i + e]);
      store16(y + row + i, v);
    }
  } else {
    for (int i = threadIdx.x; i < width; i += blockDim.x) y[row + i] = from_f32<T>(sw_row[i] * rs * next[i]);
  }
}

template <typename A> __device__ __forceinline__ float4 sw_load4(const A* p);
template <> __device__ __forceinline__ float4 sw_load4<float>(const float* p) { return *reinterpret_cast<const float4*>(p); }
template <> __device__ __forceinline__ float4 sw_load4<__nv_bfloat16>(const __nv_bfloat16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
template <typename T> __device__ __forceinline__ void sw_store4(T* p, float4 v);
template <> __device__ __forceinline__ void sw_store4<float>(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
template <> __device__ __forceinline__ void sw_store4<__nv_bfloat16>(__nv_bfloat16* p, float4 v) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<const uint32_t*>(&a);
  raw.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}
__device__ __forceinline__ float sw_dot4(float4 v) { return fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, v.w * v.w))); }

// NP packets of four entries per thread: rows of up to 1,024 * NP entries.
template <typename T, typename A, int NP>
__global__ void __launch_bounds__(256)
post_norm_add_fast_kernel(const A* __restrict__ a0, const A* __restrict__ a1, const float* __restrict__ w0,
                          const float* __restrict__ w1, int members, const float* __restrict__ post, float eps,
                          float* __restrict__ residual, float* __restrict__ results, long long result_stride, int index,
                          const float* __restrict__ coeffs, const float* __restrict__ next, T* __restrict__ y, int width) {
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();
  const size_t row = (size_t)blockIdx.x * width;
  const float inv_w = 1.0f / (float)width;
  float4 u[NP], v[NP], r[NP], s[NP];
  // everything this row reads from memory is requested here
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    const int i = (p * 256 + threadIdx.x) * 4;
    u[p] = v[p] = r[p] = s[p] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < width) {
      u[p] = sw_load4<A>(a0 + row + i);
      if (members > 1) v[p] = sw_load4<A>(a1 + row + i);
      if (post) r[p] = *reinterpret_cast<const float4*>(residual + row + i);
    }
  }
  if (results && post) {
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const int i = (p * 256 + threadIdx.x) * 4;
      if (i >= width) continue;
      const float* base = results + row + i;
      int j = 0;
      for (; j + 4 <= index; j += 4) {      // four earlier results requested together, added in ascending order
        float4 h[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) h[q] = *reinterpret_cast<const float4*>(base + (size_t)(j + q) * result_stride);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float cj = coeffs[j + q];
          s[p].x = fmaf(cj, h[q].x, s[p].x); s[p].y = fmaf(cj, h[q].y, s[p].y);
          s[p].z = fmaf(cj, h[q].z, s[p].z); s[p].w = fmaf(cj, h[q].w, s[p].w);
        }
      }
      for (; j < index; ++j) {
        const float cj = coeffs[j];
        const float4 h = *reinterpret_cast<const float4*>(base + (size_t)j * result_stride);
        s[p].x = fmaf(cj, h.x, s[p].x); s[p].y = fmaf(cj, h.y, s[p].y); s[p].z = fmaf(cj, h.z, s[p].z); s[p].w = fmaf(cj, h.w, s[p].w);
      }
    }
  }
  if (members > 0) {
    float q0 = 0.f, q1 = 0.f;
#pragma unroll
    for (int p = 0; p < NP; ++p) { q0 += sw_dot4(u[p]); q1 += sw_dot4(v[p]); }
    const float r0 = 1.0f / sqrtf(block_sum(q0, red) * inv_w + eps);
    const float r1 = members > 1 ? 1.0f / sqrtf(block_sum(q1, red) * inv_w + eps) : 0.f;
    const float share = 1.0f / (float)members;
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const int i = (p * 256 + threadIdx.x) * 4;
      if (i >= width) continue;
      const float4 wa = *reinterpret_cast<const float4*>(w0 + i);
      float4 m = make_float4(u[p].x * r0 * wa.x, u[p].y * r0 * wa.y, u[p].z * r0 * wa.z, u[p].w * r0 * wa.w);
      if (members > 1) {
        const float4 wb = *reinterpret_cast<const float4*>(w1 + i);
        m.x += v[p].x * r1 * wb.x; m.y += v[p].y * r1 * wb.y; m.z += v[p].z * r1 * wb.z; m.w += v[p].w * r1 * wb.w;
      }
      u[p] = make_float4(m.x * share, m.y * share, m.z * share, m.w * share);
    }
  }
  if (!post) {
#pragma unroll
    for (int p = 0; p < NP; ++p) {
      const int i = (p * 256 + threadIdx.x) * 4;
      if (i < width) sw_store4<T>(y + row + i, u[p]);
    }
    return;
  }
  float sq = 0.f;
#pragma unroll
  for (int p = 0; p < NP; ++p) sq += sw_dot4(u[p]);
  const float ru = 1.0f / sqrtf(block_sum(sq, red) * inv_w + eps);
  sq = 0.f;
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    const int i = (p * 256 + threadIdx.x) * 4;
    if (i >= width) continue;
    const float4 p4 = *reinterpret_cast<const float4*>(post + i);
    float4 x = make_float4(fmaf(u[p].x * ru, p4.x, r[p].x), fmaf(u[p].y * ru, p4.y, r[p].y), fmaf(u[p].z * ru, p4.z, r[p].z),
                           fmaf(u[p].w * ru, p4.w, r[p].w));
    if (results) {
      *reinterpret_cast<float4*>(results + (size_t)index * result_stride + row + i) = x;
      const float c = coeffs[index];
      x = make_float4(fmaf(c, x.x, s[p].x), fmaf(c, x.y, s[p].y), fmaf(c, x.z, s[p].z), fmaf(c, x.w, s[p].w));
    }
    *reinterpret_cast<float4*>(residual + row + i) = x;
    u[p] = x;
    sq += sw_dot4(x);
  }
  if (!next) return;
  const float rs = 1.0f / sqrtf(block_sum(sq, red) * inv_w + eps);
#pragma unroll
  for (int p = 0; p < NP; ++p) {
    const int i = (p * 256 + threadIdx.x) * 4;
    if (i >= width) continue;
    const float4 n4 = *reinterpret_cast<const float4*>(next + i);
    sw_store4<T>(y + row + i, make_float4(u[p].x * rs * n4.x, u[p].y * rs * n4.y, u[p].z * rs * n4.z, u[p].w * rs * n4.w));
  }
}

template <typename T, typename A>
int post_norm_add(const void* a0, const void* a1, const float* w0, const float* w1, int members, const float* post, float eps,
                  float* residual, float* results, long long result_stride, int index, const float* coeffs, const float* next,
                  void* y, int rows, int width, void* stream) {
  PTL_REQUIRE(rows >= 0 && width > 0 && eps > 0.f && a0, "post_norm_add: bad arguments");
  PTL_REQUIRE(members >= 0 && members <= 2 && (members < 1 || w0) && (members < 2 || (a1 && w1)),
              "post_norm_add: %d members (at most 2, each with its weight)", members);
  PTL_REQUIRE(post ? residual != nullptr : y != nullptr, "post_norm_add: nothing to write");
  PTL_REQUIRE(!results || (coeffs && index >= 0 && result_stride >= (long long)rows * width), "post_norm_add: bad results buffer");
  PTL_REQUIRE(!next || y, "post_norm_add: the next norm needs an output");
  PTL_REQUIRE((size_t)width * sizeof(float) <= 200 * 1024, "post_norm_add: rows of %d do not fit shared memory", width);
  if (rows == 0) return 0;
  // whole packets in every tensor that is walked in packets (A and T may be 2 or 4 bytes wide: 8 elements cover both)
  const int vec = width % 8 == 0 && aligned16(w0) && aligned16(w1) && aligned16(a0) && (!a1 || aligned16(a1)) && aligned16(residual) && aligned16(post) &&
                  aligned16(results) && aligned16(y) && aligned16(next) && result_stride % 4 == 0;
  if (vec && width <= 4096) {
#define PTL_SW_FAST(NP)                                                                                                         \
    return launch_kernel("post_norm_add", post_norm_add_fast_kernel<T, A, NP>, dim3(rows), dim3(256), 0, as_stream(stream),       \
                         (const A*)a0, (const A*)a1, w0, w1, members, post, eps, residual, results, result_stride, index, coeffs, \
                         next, (T*)y, width)
    if (width <= 1024) PTL_SW_FAST(1);
    if (width <= 2048) PTL_SW_FAST(2);
    PTL_SW_FAST(4);
#undef PTL_SW_FAST
  }
  const size_t smem = (size_t)width * sizeof(float);
  static SmemRaised raised;
  if (smem > 48 * 1024)
    if (int rc = raise_shared_memory("post_norm_add", post_norm_add_kernel<T, A>, 200 * 1024, raised)) return rc;
  return launch_kernel("post_norm_add", post_norm_add_kernel<T, A>, dim3(rows), dim3(256), smem, as_stream(stream), (const A*)a0,
                       (const A*)a1, w0, w1, members, post, eps, residual, results, result_stride, index, coeffs, next, (T*)y,
                       width, vec);
}

}  // namespace ptl

// a_f32: the sub-layer outputs are float32 whatever the compute type
#define PTL_SANDWICH(SUFFIX, TYPE)                                                                                                \
  PTL_EXPORT int ptl_post_norm_add##SUFFIX(const void* a0, const void* a1, const float* w0, const float* w1, int members,          \
                                           const float* post, float eps, float* residual, float* results, long long result_stride, \
                                           int index, const float* coeffs, const float* next, void* y, int rows, int width,       \
                                           int a_f32, void* stream) {                                                             \
    if (a_f32)                                                                                                                    \
      return ptl::post_norm_add<TYPE, float>(a0, a1, w0, w1, members, post, eps, residual, results, result_stride, index, coeffs, \
                                             next, y, rows, width, stream);                                                       \
    return ptl::post_norm_add<TYPE, TYPE>(a0, a1, w0, w1, members, post, eps, residual, results, result_stride, index, coeffs,     \
                                          next, y, rows, width, stream);                                                          \
  }
PTL_SANDWICH(_f32, float)
PTL_SANDWICH(_bf16, __nv_bfloat16)
