// Inputs of the attention through latents (parts/latent_attention.py).
//
// latent_norm_store, per token, on the projection's output [T, q latent (Q) | kv latent (R) | rotated key part (n) | ...]:
//   cq = q latent * rsqrt(mean(q latent^2) + eps) * wq          -> out_q [T, Q]
//   c  = kv latent * rsqrt(mean(kv latent^2) + eps) * wkv       (R > 0 only)
//   k_r = the n entries after the kv latent, pairs (2i, 2i+1), i < dims/2, turned by float(position) * freq[i]
//   [c | k_r], rounded once, goes to the token's slot of a cache whose pages hold keys of R + n entries and nothing else.
// Sums of squares, the norms and the angles are float32.
//
// rotate_head_part, per token and head: n entries at column x_col of a head of x (rows of heads * x_ld) are copied to
// column out_col of the same head of out (rows of heads * out_ld), the pairs (2i, 2i+1), i < dims/2, turned likewise.
#include "common.cuh"

namespace ptl {

template <typename T>
__global__ void __launch_bounds__(256)
latent_norm_store_kernel(T* __restrict__ out_q, const T* __restrict__ proj, int ld, int Q, const float* __restrict__ wq, int R,
                         const float* __restrict__ wkv, int n, float eps, const int* __restrict__ positions,
                         const float* __restrict__ freq, int dims, const int* __restrict__ slots, T* __restrict__ cache,
                         long long num_slots) {
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const T* row = proj + (size_t)t * ld;
  float sq = 0.f;
  for (int i = threadIdx.x; i < Q; i += blockDim.x) { const float v = to_f32(row[i]); sq = fmaf(v, v, sq); }
  sq = block_sum(sq, red);
  const float rq = 1.0f / sqrtf(sq / (float)Q + eps);
  for (int i = threadIdx.x; i < Q; i += blockDim.x) out_q[(size_t)t * Q + i] = from_f32<T>(to_f32(row[i]) * rq * wq[i]);
  if (R <= 0) return;
  float sk = 0.f;
  for (int i = threadIdx.x; i < R; i += blockDim.x) { const float v = to_f32(row[Q + i]); sk = fmaf(v, v, sk); }
  sk = block_sum(sk, red);
  const float rk = 1.0f / sqrtf(sk / (float)R + eps);
  long long slot = (slots && cache) ? (long long)slots[t] : -1;
  if (slot < 0 || slot >= num_slots) return;
  T* dst = cache + (size_t)slot * (R + n);
  for (int i = threadIdx.x; i < R; i += blockDim.x) dst[i] = from_f32<T>(to_f32(row[Q + i]) * rk * wkv[i]);
  const float pos = (float)positions[t];
  const T* kr = row + Q + R;
  for (int i = threadIdx.x; i < (n + 1) / 2; i += blockDim.x) {
    const int e0 = 2 * i, e1 = 2 * i + 1;
    float a = to_f32(kr[e0]), b = e1 < n ? to_f32(kr[e1]) : 0.f;
    if (e1 < dims) {
      float sn, cs, o1, o2;
      sincosf(pos * freq[i], &sn, &cs);
      rope_rotate(a, b, cs, sn, o1, o2);
      a = o1;
      b = o2;
    }
    dst[R + e0] = from_f32<T>(a);
    if (e1 < n) dst[R + e1] = from_f32<T>(b);
  }
}

template <typename T>
__global__ void __launch_bounds__(128)
rotate_head_part_kernel(T* __restrict__ out, int out_ld, int out_col, const T* __restrict__ x, int x_ld, int x_col, int heads, int n,
                        const int* __restrict__ positions, const float* __restrict__ freq, int dims) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const float pos = (float)positions[t];
  const int pairs = (n + 1) / 2;
  for (int idx = threadIdx.x; idx < heads * pairs; idx += blockDim.x) {
    const int h = idx / pairs, i = idx % pairs;
    const int e0 = 2 * i, e1 = 2 * i + 1;
    const T* src = x + (size_t)t * heads * x_ld + (size_t)h * x_ld + x_col;
    T* dst = out + (size_t)t * heads * out_ld + (size_t)h * out_ld + out_col;
    float a = to_f32(src[e0]), b = e1 < n ? to_f32(src[e1]) : 0.f;
    if (e1 < dims) {
      float sn, cs, o1, o2;
      sincosf(pos * freq[i], &sn, &cs);
      rope_rotate(a, b, cs, sn, o1, o2);
      a = o1;
      b = o2;
    }
    dst[e0] = from_f32<T>(a);
    if (e1 < n) dst[e1] = from_f32<T>(b);
  }
}

template <typename T>
int latent_norm_store(void* out_q, const void* proj, int tokens, int ld, int Q, const float* wq, int R, const float* wkv, int n,
                      float eps, const int* positions, const float* freq, int dims, const int* slots, void* cache,
                      long long num_slots, void* stream) {
  PTL_REQUIRE(tokens >= 0 && Q > 0 && R >= 0 && n >= 0 && eps > 0.f && wq && ld >= Q + R + (R > 0 ? n : 0),
              "latent_norm_store: bad sizes Q=%d R=%d n=%d ld=%d", Q, R, n, ld);
  PTL_REQUIRE(R == 0 || (wkv && positions && dims >= 0 && dims % 2 == 0 && dims <= n && (dims == 0 || freq)),
              "latent_norm_store: the kept part needs its norm weight, positions and %d <= %d rotated entries", dims, n);
  if (tokens == 0) return 0;
  return launch_kernel("latent_norm_store", latent_norm_store_kernel<T>, dim3(tokens), dim3(256), 0, as_stream(stream), (T*)out_q,
                       (const T*)proj, ld, Q, wq, R, wkv, n, eps, positions, freq, dims, slots, (T*)cache, num_slots);
}

template <typename T>
int rotate_head_part(void* out, int out_ld, int out_col, const void* x, int x_ld, int x_col, int tokens, int heads, int n,
                     const int* positions, const float* freq, int dims, void* stream) {
  PTL_REQUIRE(tokens >= 0 && heads > 0 && n > 0 && x_col >= 0 && x_col + n <= x_ld && out_col >= 0 && out_col + n <= out_ld &&
              dims >= 0 && dims % 2 == 0 && dims <= n && (dims == 0 || freq), "rotate_head_part: bad sizes");
  if (tokens == 0) return 0;
  return launch_kernel("rotate_head_part", rotate_head_part_kernel<T>, dim3(tokens), dim3(128), 0, as_stream(stream), (T*)out, out_ld,
                       out_col, (const T*)x, x_ld, x_col, heads, n, positions, freq, dims);
}

}  // namespace ptl

#define PTL_LATENT(SUFFIX, TYPE)                                                                                                  \
  PTL_EXPORT int ptl_latent_norm_store##SUFFIX(void* out_q, const void* proj, int tokens, int ld, int Q, const float* wq, int R,   \
                                               const float* wkv, int n, float eps, const int* positions, const float* freq,       \
                                               int dims, const int* slots, void* cache, long long num_slots, void* stream) {      \
    return ptl::latent_norm_store<TYPE>(out_q, proj, tokens, ld, Q, wq, R, wkv, n, eps, positions, freq, dims, slots, cache,       \
                                        num_slots, stream);                                                                       \
  }                                                                                                                               \
  PTL_EXPORT int ptl_rotate_head_part##SUFFIX(void* out, int out_ld, int out_col, const void* x, int x_ld, int x_col, int tokens,  \
                                              int heads, int n, const int* positions, const float* freq, int dims, void* stream) { \
    return ptl::rotate_head_part<TYPE>(out, out_ld, out_col, x, x_ld, x_col, tokens, heads, n, positions, freq, dims, stream);     \
  }
PTL_LATENT(_f32, float)
PTL_LATENT(_bf16, __nv_bfloat16)
