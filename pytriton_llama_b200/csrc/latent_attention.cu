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
//
// For prompt portions the attention over the latents is made of matrix products (ops/cuda.py, latent_prefill_attention):
// latent_gather copies one request's kept rows [c | k_r] out of its pages into consecutive rows, and the latents c once
// more with keys along the rows (the second product's right operand); causal_softmax_rows turns a float32 block of
// scores, one row per (token, head), into the weights of the keys up to the token's own position (float32 maximum, sum
// and quotient; rounded once) and zeros beyond.
#include "common.cuh"

namespace ptl {

// keys [c_pad, d] and latents_t [R, c_pad] of the request whose block table row is bt: key j < ctx comes from its page,
// rows and columns from ctx to c_pad are zero.  One block per 32 keys; the tile passes shared memory so that both
// copies are written along their rows.
template <typename T>
__global__ void __launch_bounds__(256)
latent_gather_kernel(T* __restrict__ keys, T* __restrict__ latents_t, const T* __restrict__ cache, const int* __restrict__ bt,
                     int ctx, int c_pad, int d, int R, int page_size, int num_pages, int vec_ok) {
  extern __shared__ __align__(16) unsigned char lg_raw[];
  T* tile = reinterpret_cast<T*>(lg_raw);          // [32][d + 2]
  pdl_wait();
  pdl_launch_dependents();
  const int ld = d + 2;
  const int k0 = blockIdx.x * 32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (vec_ok) {
    // 16-bit entries, rows of whole packets of 16 bytes: a packet per load, four words per store into the tile (its rows
    // start on 4-byte boundaries only); then two keys of one latent entry per store, 16 lanes a row of the tile
    const int ppr = d / 8;
    for (int idx = threadIdx.x; idx < 32 * ppr; idx += blockDim.x) {
      const int row = idx / ppr, pk = idx % ppr;
      const int key = k0 + row;
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (key < ctx) {
        const int page = bt[key / page_size];
        if (page >= 0 && page < num_pages)
          v = reinterpret_cast<const uint4*>(cache + ((size_t)page * page_size + key % page_size) * d)[pk];
      }
      unsigned* tw = reinterpret_cast<unsigned*>(tile + row * ld + 8 * pk);
      tw[0] = v.x; tw[1] = v.y; tw[2] = v.z; tw[3] = v.w;
      if (key < c_pad) reinterpret_cast<uint4*>(keys + (size_t)key * d)[pk] = v;
    }
    __syncthreads();
    const int q = lane & 15, half = lane >> 4;
    if (k0 + 2 * q + 1 < c_pad) {
      for (int e = 2 * warp + half; e < R; e += 16) {
        T two[2] = {tile[(2 * q) * ld + e], tile[(2 * q + 1) * ld + e]};
        *reinterpret_cast<unsigned*>(latents_t + (size_t)e * c_pad + k0 + 2 * q) = *reinterpret_cast<unsigned*>(two);
      }
    }
    return;
  }
  for (int idx = threadIdx.x; idx < 32 * d; idx += blockDim.x) {
    const int row = idx / d, e = idx % d;
    const int key = k0 + row;
    T v = from_f32<T>(0.f);
    if (key < ctx) {
      const int page = bt[key / page_size];
      if (page >= 0 && page < num_pages) v = cache[((size_t)page * page_size + key % page_size) * d + e];
    }
    tile[row * ld + e] = v;
    if (key < c_pad) keys[(size_t)key * d + e] = v;
  }
  __syncthreads();
  if (k0 + lane < c_pad)
    for (int e = warp; e < R; e += 8) latents_t[(size_t)e * c_pad + k0 + lane] = tile[lane * ld + e];
}

// weights[row, j] = exp(scale * s[row, j] - m) / sum for j <= position of the row's token (j < n_keys), 0 for the other
// j < ld_out; with `sink` the sum has one more term exp(0 - m).  Row = token * heads + head.  One block per row.
template <typename T>
__global__ void __launch_bounds__(256)
causal_softmax_rows_kernel(T* __restrict__ weights, int ld_out, const float* __restrict__ scores, int n_keys,
                           const int* __restrict__ positions, int heads, float scale, int sink, int held) {
  extern __shared__ __align__(16) float sr_row[];     // held: the row's scaled scores, then its exponentials
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();
  const size_t row = blockIdx.x;
  const int p = positions[row / heads];
  const int n = min(p + 1, n_keys);
  const float* s = scores + row * (size_t)n_keys;
  T* w = weights + row * (size_t)ld_out;
  float m = sink ? 0.f : -INFINITY;
  if (held) {
    // n_keys and ld_out are multiples of 4 and the row fits shared memory: the scores are read once, four at a time, and
    // every exponential is worked out once.  A thread meets the same j in every pass.
    const int n4 = (n + 3) & ~3;
    for (int j = 4 * threadIdx.x; j < n4; j += 4 * blockDim.x) {
      float4 v = *reinterpret_cast<const float4*>(s + j);
      v.x *= scale; v.y *= scale; v.z *= scale; v.w *= scale;
      if (j + 1 >= n) v.y = -INFINITY;
      if (j + 2 >= n) v.z = -INFINITY;
      if (j + 3 >= n) v.w = -INFINITY;
      *reinterpret_cast<float4*>(sr_row + j) = v;
      m = fmaxf(m, fmaxf(fmaxf(v.x, v.y), fmaxf(v.z, v.w)));
    }
    m = block_max(m, red);
    float sum = 0.f;
    for (int j = 4 * threadIdx.x; j < n4; j += 4 * blockDim.x) {
      float4 v = *reinterpret_cast<const float4*>(sr_row + j);
      v.x = expf(v.x - m); v.y = expf(v.y - m); v.z = expf(v.z - m); v.w = expf(v.w - m);     // exp(-inf) = 0 beyond n
      *reinterpret_cast<float4*>(sr_row + j) = v;
      sum += (v.x + v.y) + (v.z + v.w);
    }
    sum = block_sum(sum, red);
    if (sink) sum += expf(-m);
    const float inv = sum > 0.f ? 1.0f / sum : 0.f;
    for (int j = 4 * threadIdx.x; j < ld_out; j += 4 * blockDim.x) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (j < n4) v = *reinterpret_cast<const float4*>(sr_row + j);
      T o[4] = {from_f32<T>(v.x * inv), from_f32<T>(v.y * inv), from_f32<T>(v.z * inv), from_f32<T>(v.w * inv)};
      if (sizeof(T) == 2) *reinterpret_cast<uint2*>(w + j) = *reinterpret_cast<uint2*>(o);
      else *reinterpret_cast<uint4*>(w + j) = *reinterpret_cast<uint4*>(o);
    }
    return;
  }
  for (int j = threadIdx.x; j < n; j += blockDim.x) m = fmaxf(m, s[j] * scale);
  m = block_max(m, red);
  float sum = 0.f;
  for (int j = threadIdx.x; j < n; j += blockDim.x) sum += expf(s[j] * scale - m);
  sum = block_sum(sum, red);
  if (sink) sum += expf(-m);
  const float inv = sum > 0.f ? 1.0f / sum : 0.f;
  for (int j = threadIdx.x; j < ld_out; j += blockDim.x) w[j] = from_f32<T>(j < n ? expf(s[j] * scale - m) * inv : 0.f);
}

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

template <typename T>
int latent_gather(void* keys, void* latents_t, const void* cache, const int* bt, int ctx, int c_pad, int d, int R, int page_size,
                  int num_pages, void* stream) {
  PTL_REQUIRE(ctx >= 0 && c_pad >= ctx && d > 0 && R > 0 && R <= d && page_size > 0 && num_pages > 0, "latent_gather: bad sizes");
  const size_t smem = (size_t)32 * (d + 2) * sizeof(T);
  PTL_REQUIRE(smem <= 48 * 1024, "latent_gather: rows of %d entries do not fit shared memory", d);
  if (c_pad == 0) return 0;
  const int vec_ok = sizeof(T) == 2 && d % 8 == 0 && c_pad % 2 == 0 && aligned16(keys) && aligned16(cache) &&
                     (reinterpret_cast<uintptr_t>(latents_t) & 3u) == 0;
  return launch_kernel("latent_gather", latent_gather_kernel<T>, dim3((c_pad + 31) / 32), dim3(256), smem, as_stream(stream),
                       (T*)keys, (T*)latents_t, (const T*)cache, bt, ctx, c_pad, d, R, page_size, num_pages, vec_ok);
}

template <typename T>
int causal_softmax_rows(void* weights, int ld_out, const float* scores, long long rows, int n_keys, const int* positions,
                        int heads, float scale, int sink, void* stream) {
  PTL_REQUIRE(rows >= 0 && rows < (1ll << 31) && n_keys > 0 && ld_out >= n_keys && heads > 0, "causal_softmax_rows: bad sizes");
  if (rows == 0) return 0;
  const int held = n_keys % 4 == 0 && ld_out % 4 == 0 && (size_t)n_keys * sizeof(float) <= 40 * 1024 && aligned16(scores) &&
                   aligned16(weights);
  return launch_kernel("causal_softmax_rows", causal_softmax_rows_kernel<T>, dim3((unsigned)rows), dim3(256),
                       held ? (size_t)n_keys * sizeof(float) : 0, as_stream(stream), (T*)weights, ld_out, scores, n_keys, positions,
                       heads, scale, sink, held);
}

// out[t, h * ld + col + c] *= sigmoid(gate[t * gate_ld + h]), c < n (float32 inside, rounded once): the heads' gates on a
// result that a batched product of the library wrote.  One block per token.
template <typename T>
__global__ void __launch_bounds__(256)
head_gate_kernel(T* __restrict__ out, int ld, int col, int n, int heads, const T* __restrict__ gate, int gate_ld) {
  pdl_wait();
  pdl_launch_dependents();
  const size_t t = blockIdx.x;
  for (int idx = threadIdx.x; idx < heads * n; idx += blockDim.x) {
    const int h = idx / n, c = idx % n;
    const float g = 1.0f / (1.0f + expf(-to_f32(gate[t * gate_ld + h])));
    T* o = out + t * (size_t)heads * ld + (size_t)h * ld + col + c;
    *o = from_f32<T>(to_f32(*o) * g);
  }
}

template <typename T>
int head_gate(void* out, int ld, int col, int n, int tokens, int heads, const void* gate, int gate_ld, void* stream) {
  PTL_REQUIRE(tokens >= 0 && heads > 0 && n > 0 && col >= 0 && col + n <= ld && gate && gate_ld >= heads, "head_gate: bad sizes");
  if (tokens == 0) return 0;
  return launch_kernel("head_gate", head_gate_kernel<T>, dim3(tokens), dim3(256), 0, as_stream(stream), (T*)out, ld, col, n, heads,
                       (const T*)gate, gate_ld);
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
  }                                                                                                                               \
  PTL_EXPORT int ptl_head_gate##SUFFIX(void* out, int ld, int col, int n, int tokens, int heads, const void* gate, int gate_ld,    \
                                       void* stream) {                                                                            \
    return ptl::head_gate<TYPE>(out, ld, col, n, tokens, heads, gate, gate_ld, stream);                                           \
  }
#define PTL_LATENT_PREFILL(SUFFIX, TYPE)                                                                                          \
  PTL_EXPORT int ptl_latent_gather##SUFFIX(void* keys, void* latents_t, const void* cache, const int* bt, int ctx, int c_pad,      \
                                           int d, int R, int page_size, int num_pages, void* stream) {                           \
    return ptl::latent_gather<TYPE>(keys, latents_t, cache, bt, ctx, c_pad, d, R, page_size, num_pages, stream);                  \
  }                                                                                                                               \
  PTL_EXPORT int ptl_causal_softmax_rows##SUFFIX(void* weights, int ld_out, const float* scores, long long rows, int n_keys,       \
                                                 const int* positions, int heads, float scale, int sink, void* stream) {          \
    return ptl::causal_softmax_rows<TYPE>(weights, ld_out, scores, rows, n_keys, positions, heads, scale, sink, stream);          \
  }
PTL_LATENT_PREFILL(_f32, float)
PTL_LATENT_PREFILL(_bf16, __nv_bfloat16)
PTL_LATENT(_f32, float)
PTL_LATENT(_bf16, __nv_bfloat16)
