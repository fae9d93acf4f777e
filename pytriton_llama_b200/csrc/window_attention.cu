// Softmax attention behind a sliding window that keeps the first positions, over the paged cache,
// and the kernel that prepares its inputs.
//
// A page of the cache holds its keys, then its values: key n of kv head g lies at
//   page * G * page_size * (d + dv) + (g * page_size + n % page_size) * d,
// its value at  page * G * page_size * (d + dv) + G * page_size * d + (g * page_size + n % page_size) * dv.
// (With dv == d this is the [pages][2][G][page_size][d] layout of the other attention kernels.)
//
// qk_norm_rotate_store, per token of the step, on the projection's output [T, q | k | v]:
//   q <- q * rsqrt(mean(q^2) + eps) * wq   over ALL heads of the token at once; k likewise     (eps > 0)
//   pairs (2i, 2i+1), i < dims/2, of every q and k head are turned by the angle float(position) * freq[i],
//   cos and sin multiplied by `amplitude`;
//   q and k are written back in place (rounded once), k and v go to the token's slot of the cache.
//
// window_attention: token t (request r, position p) sees key j <= p if p - j < window or j < keep
// (window 0: every j <= p).  One warp per (token, query head); the visible keys are walked as one
// list (the kept ones that the window has passed, then the window), 32 at a time, one key per
// lane; scores, softmax and the weighted sum of values are float32, with float32 inputs compensated
// (see attention_simt.cu).  The list may be split over blockIdx.z and merged by a second kernel.
// The kernel works `tokens` rows, or the rows that `items` names (the single tokens of a step
// whose longer portions another kernel takes); partial results are indexed by the row itself.
// Options: `sink` adds one term of score 0 (and no value) to the softmax's denominator; `temp_coef` != 0
// multiplies the scores of the query at position p by 1 + temp_coef * ln(floor((p + 1) / temp_every) + 1);
// `shared_v`: pages hold keys only and the value of a key is its first dv entries.  `bias_exp` = c > 0: head h takes
// 2^(-c (h + 1) / H) * (p - j) off the score of key j.  `gate_col` >= 0: the result of head h is multiplied by the
// sigmoid of the dv entries at column gate_col + h * dv of the token's q row.  `pool` = P > 0 (with a window): the list
// starts with one mean key and mean value for every block b of P positions with bP + P - 1 <= p - window, read from
// `summary`, pages of the cache's layout with a block table of their own; that part of the list is padded to whole
// turns of 32 so that a turn reads either means or tokens.
//
// head_norm_rotate_store, per token, on [T, q | k | v | ...]: every q and k head divided by its own root mean square
// and multiplied by the weight [d] of its kind (eps > 0), entries i and i + rot/2 of a head turned by
// position * inv_freq[i] (the table float32 or float64, the product and its sine and cosine in 64 bits, once per token
// and pair); in place, k and v to the token's slot.  A warp per head.
//
// pool_blocks, per token with a slot in `summary`: the mean over the P positions that end with the token's own of
// the keys and of the values in the cache, added in ascending order of position and divided by P.
#include "common.cuh"

namespace ptl {

// ------------------------------------------------------------------ norm + rotation + cache write
template <typename T>
__global__ void __launch_bounds__(256)
qk_norm_rotate_store_kernel(T* __restrict__ proj, int ld, int H, int G, int d, int dv, const float* __restrict__ wq,
                            const float* __restrict__ wk, float eps, const int* __restrict__ positions,
                            const float* __restrict__ freq, int dims, float amplitude, const int* __restrict__ slots,
                            T* __restrict__ cache, int page_size, long long num_slots, int vec_ok) {
  __shared__ float red[33];
  __shared__ float s_cs[256], s_sn[256];          // cos and sin (times the amplitude) of the token's angles, vec_ok only
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  T* row = proj + (size_t)t * ld;
  const int nq = H * d, nk = G * d, nv = G * dv;
  float rq = 1.f, rk = 1.f;
  constexpr int VN = Vec16<T>::N;
  if (vec_ok) {
    // Packets of 16 bytes: the sums of squares, then every packet of q and k (it lies within one head) normed, turned
    // by angles worked out once per token, written back and, for k, stored; v is copied packet by packet.
    const float pos = (float)positions[t];
    if (freq && threadIdx.x < dims / 2) {
      float sn, cs;
      sincosf(pos * freq[threadIdx.x], &sn, &cs);
      s_cs[threadIdx.x] = cs * amplitude;
      s_sn[threadIdx.x] = sn * amplitude;
    }
    float sq = 0.f, sk = 0.f;
    if (eps > 0.f) {
      for (int i = threadIdx.x * VN; i < nq + nk; i += blockDim.x * VN) {
        const Vec16<T> v = load16(row + i);
        float part = 0.f;
#pragma unroll
        for (int e = 0; e < VN; ++e) part = fmaf(v.get(e), v.get(e), part);
        if (i < nq) sq += part; else sk += part;
      }
      sq = block_sum(sq, red);
      rq = 1.0f / sqrtf(sq / (float)nq + eps);
      if (nk > 0) {
        sk = block_sum(sk, red);
        rk = 1.0f / sqrtf(sk / (float)nk + eps);
      }
    } else {
      __syncthreads();
    }
    long long slot = (slots && cache) ? (long long)slots[t] : -1;
    if (slot >= num_slots) slot = -1;
    const size_t page_stride = (size_t)G * page_size * (d + dv);
    const size_t page = slot >= 0 ? (size_t)(slot / page_size) : 0, off = slot >= 0 ? (size_t)(slot % page_size) : 0;
    for (int i = threadIdx.x * VN; i < nq + nk; i += blockDim.x * VN) {
      const bool is_k = i >= nq;
      const int within = (is_k ? i - nq : i) % d;          // first entry of the packet within its head
      const float r = is_k ? rk : rq;
      Vec16<T> v = load16(row + i);
      float x[VN];
#pragma unroll
      for (int e = 0; e < VN; ++e) x[e] = v.get(e) * r;
      if (eps > 0.f) {
        const float* w = is_k ? wk + (i - nq) : wq + i;
#pragma unroll
        for (int e = 0; e < VN; ++e) x[e] *= w[e];
      }
      if (freq && within < dims) {
#pragma unroll
        for (int e = 0; e < VN; e += 2) {
          if (within + e + 1 < dims) {
            const int pair = (within + e) >> 1;
            float o1, o2;
            rope_rotate(x[e], x[e + 1], s_cs[pair], s_sn[pair], o1, o2);
            x[e] = o1;
            x[e + 1] = o2;
          }
        }
      }
#pragma unroll
      for (int e = 0; e < VN; ++e) v.set(e, x[e]);
      store16(row + i, v);
      if (is_k && slot >= 0) {
        const int g = (i - nq) / d;
        store16(cache + page * page_stride + ((size_t)g * page_size + off) * d + within, v);
      }
    }
    if (slot >= 0) {
      const T* vsrc = row + nq + nk;
      T* vdst = cache + page * page_stride + (size_t)G * page_size * d + off * dv;
      for (int i = threadIdx.x * VN; i < nv; i += blockDim.x * VN) {
        const int g = i / dv, e = i % dv;
        store16(vdst + (size_t)g * page_size * dv + e, load16(vsrc + i));
      }
    }
    return;
  }
  if (eps > 0.f) {
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < nq; i += blockDim.x) { const float v = to_f32(row[i]); sq = fmaf(v, v, sq); }
    for (int i = threadIdx.x; i < nk; i += blockDim.x) { const float v = to_f32(row[nq + i]); sk = fmaf(v, v, sk); }
    sq = block_sum(sq, red);
    rq = 1.0f / sqrtf(sq / (float)nq + eps);
    if (nk > 0) {
      sk = block_sum(sk, red);
      rk = 1.0f / sqrtf(sk / (float)nk + eps);
    }
  }
  const float pos = (float)positions[t];
  long long slot = (slots && cache) ? (long long)slots[t] : -1;
  if (slot >= num_slots) slot = -1;
  const size_t page_stride = (size_t)G * page_size * (d + dv);
  T* kdst = nullptr;
  T* vdst = nullptr;
  if (slot >= 0) {
    const size_t page = (size_t)(slot / page_size), off = (size_t)(slot % page_size);
    kdst = cache + page * page_stride + off * d;                                  // + g * page_size * d
    vdst = cache + page * page_stride + (size_t)G * page_size * d + off * dv;     // + g * page_size * dv
  }
  // q and k, two neighbours per thread and turn (d is even when anything is rotated; an odd last entry is handled alone)
  const int heads = H + G;
  const int pairs_per_head = (d + 1) / 2;
  for (int idx = threadIdx.x; idx < heads * pairs_per_head; idx += blockDim.x) {
    const int h = idx / pairs_per_head, i = idx % pairs_per_head;
    const int e0 = 2 * i, e1 = 2 * i + 1;
    const bool is_k = h >= H;
    const float r = is_k ? rk : rq;
    const float* w = eps > 0.f ? (is_k ? wk + (size_t)(h - H) * d : wq + (size_t)h * d) : nullptr;
    T* src = row + (size_t)h * d;
    float a = to_f32(src[e0]) * r * (w ? w[e0] : 1.f);
    float b = e1 < d ? to_f32(src[e1]) * r * (w ? w[e1] : 1.f) : 0.f;
    if (freq && e1 < dims) {
      float sn, cs;
      sincosf(pos * freq[i], &sn, &cs);
      float o1, o2;
      rope_rotate(a, b, cs * amplitude, sn * amplitude, o1, o2);
      a = o1;
      b = o2;
    }
    const T ta = from_f32<T>(a), tb = from_f32<T>(b);
    src[e0] = ta;
    if (e1 < d) src[e1] = tb;
    if (is_k && kdst) {
      T* kd = kdst + (size_t)(h - H) * page_size * d;
      kd[e0] = ta;
      if (e1 < d) kd[e1] = tb;
    }
  }
  if (vdst) {
    const T* v = row + nq + nk;
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
      const int g = i / dv, e = i % dv;
      vdst[(size_t)g * page_size * dv + e] = v[i];
    }
  }
}

template <typename T>
int qk_norm_rotate_store(void* proj, int tokens, int ld, int H, int G, int d, int dv, const float* wq, const float* wk, float eps,
                         const int* positions, const float* freq, int dims, float amplitude, const int* slots, void* cache,
                         int page_size, long long num_slots, void* stream) {
  PTL_REQUIRE(tokens >= 0 && H > 0 && G >= 0 && d > 0 && dv > 0 && page_size > 0, "qk_norm_rotate_store: bad sizes");
  PTL_REQUIRE(ld >= H * d + G * (d + dv), "qk_norm_rotate_store: rows of %d elements are too short", ld);
  PTL_REQUIRE(eps <= 0.f || (wq && (G == 0 || wk)), "qk_norm_rotate_store: the norm needs its weights");
  PTL_REQUIRE(dims >= 0 && dims % 2 == 0 && dims <= d && (dims == 0 || freq), "qk_norm_rotate_store: rotary width %d of head size %d", dims, d);
  if (tokens == 0) return 0;
  constexpr int VN = Vec16<T>::N;
  const int vec_ok = d % VN == 0 && dv % VN == 0 && ld % VN == 0 && dims <= 512 && aligned16(proj) &&
                     (!cache || aligned16(cache)) && (eps <= 0.f || (aligned16(wq) && (G == 0 || aligned16(wk))));
  return launch_kernel("qk_norm_rotate_store", qk_norm_rotate_store_kernel<T>, dim3(tokens), dim3(256), 0, as_stream(stream),
                       (T*)proj, ld, H, G, d, dv, wq, wk, eps, positions, dims > 0 ? freq : nullptr, dims, amplitude,
                       G > 0 ? slots : nullptr, (T*)cache, page_size, num_slots, vec_ok);
}

// ------------------------------------------------------------------ per-head norm + rotation of halves + cache write
template <typename T>
__global__ void __launch_bounds__(256)
head_norm_rotate_store_kernel(T* __restrict__ proj, int ld, int H, int G, int d, int dv, const float* __restrict__ wq,
                              const float* __restrict__ wk, float eps, const int* __restrict__ positions,
                              const void* __restrict__ inv_freq, int freq64, int rot, const int* __restrict__ slots,
                              T* __restrict__ cache, int page_size, long long num_slots) {
  extern __shared__ float hn_smem[];       // cos[rot/2], sin[rot/2], then d floats per warp
  const int t = blockIdx.x;
  const int half = rot / 2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  float* cs = hn_smem;
  float* sn = hn_smem + half;
  float* buf = hn_smem + 2 * half + warp * d;
  // (the angle itself in 64 bits: a float32 product of a position in the thousands and a frequency is off by up to
  // 1e-4 radians, which float32 logits show; this runs once per token and pair)
  const double pos = (double)positions[t];   // an input of the step, not a result of the kernel before
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    double s64, c64;
    const double f = freq64 ? reinterpret_cast<const double*>(inv_freq)[j] : (double)reinterpret_cast<const float*>(inv_freq)[j];
    sincos(pos * f, &s64, &c64);
    sn[j] = (float)s64;
    cs[j] = (float)c64;
  }
  pdl_wait();
  pdl_launch_dependents();
  __syncthreads();
  T* row = proj + (size_t)t * ld;
  long long slot = (slots && cache) ? (long long)slots[t] : -1;
  if (slot >= num_slots) slot = -1;
  const size_t page_stride = (size_t)G * page_size * (d + dv);
  T* kdst = nullptr;
  T* vdst = nullptr;
  if (slot >= 0) {
    const size_t page = (size_t)(slot / page_size), off = (size_t)(slot % page_size);
    kdst = cache + page * page_stride + off * d;                                  // + g * page_size * d
    vdst = cache + page * page_stride + (size_t)G * page_size * d + off * dv;     // + g * page_size * dv
  }
  for (int h = warp; h < H + G; h += nwarps) {
    T* src = row + (size_t)h * d;
    const bool is_k = h >= H;
    float ss = 0.f;
    for (int i = lane; i < d; i += 32) {
      const float v = to_f32(src[i]);
      buf[i] = v;
      ss = fmaf(v, v, ss);
    }
    float r = 1.f;
    if (eps > 0.f) r = 1.0f / sqrtf(warp_sum(ss) / (float)d + eps);
    __syncwarp();
    const float* w = eps > 0.f ? (is_k ? wk : wq) : nullptr;
    T* kd = (is_k && kdst) ? kdst + (size_t)(h - H) * page_size * d : nullptr;
    for (int i = lane; i < d; i += 32) {
      float x = buf[i] * r * (w ? w[i] : 1.f);
      if (i < rot) {
        const int j = i < half ? i : i - half;
        const int other = i < half ? i + half : i - half;
        const float xo = buf[other] * r * (w ? w[other] : 1.f);
        x = i < half ? fmaf(x, cs[j], -xo * sn[j]) : fmaf(x, cs[j], xo * sn[j]);
      }
      const T o = from_f32<T>(x);
      src[i] = o;
      if (kd) kd[i] = o;
    }
    __syncwarp();
  }
  if (vdst) {
    const T* v = row + (size_t)(H + G) * d;
    for (int i = threadIdx.x; i < G * dv; i += blockDim.x) {
      const int g = i / dv, e = i % dv;
      vdst[(size_t)g * page_size * dv + e] = v[i];
    }
  }
}

template <typename T>
int head_norm_rotate_store(void* proj, int tokens, int ld, int H, int G, int d, int dv, const float* wq, const float* wk, float eps,
                           const int* positions, const void* inv_freq, int freq64, int rot, const int* slots, void* cache,
                           int page_size, long long num_slots, void* stream) {
  PTL_REQUIRE(tokens >= 0 && H > 0 && G >= 0 && d > 0 && dv > 0 && page_size > 0, "head_norm_rotate_store: bad sizes");
  PTL_REQUIRE(ld >= (H + G) * d + G * dv, "head_norm_rotate_store: rows of %d elements are too short", ld);
  PTL_REQUIRE(eps <= 0.f || (wq && (G == 0 || wk)), "head_norm_rotate_store: the norm needs its weights");
  PTL_REQUIRE(rot >= 0 && rot % 2 == 0 && rot <= d && (rot == 0 || inv_freq), "head_norm_rotate_store: rotary width %d of head size %d", rot, d);
  PTL_REQUIRE(d <= 4096, "head_norm_rotate_store: head size %d", d);
  if (tokens == 0) return 0;
  const size_t smem = ((size_t)rot + 8 * (size_t)d) * sizeof(float);
  static SmemRaised raised;
  if (smem > 48 * 1024)
    if (int rc = raise_shared_memory("head_norm_rotate_store", head_norm_rotate_store_kernel<T>, 200 * 1024, raised)) return rc;
  return launch_kernel("head_norm_rotate_store", head_norm_rotate_store_kernel<T>, dim3(tokens), dim3(256), smem, as_stream(stream),
                       (T*)proj, ld, H, G, d, dv, wq, wk, eps, positions, rot > 0 ? inv_freq : nullptr, freq64, rot,
                       G > 0 ? slots : nullptr, (T*)cache, page_size, num_slots);
}

// ------------------------------------------------------------------ means of whole blocks
constexpr int kPoolStaged = 256;      // positions of a block whose rows are looked up once and kept in shared memory

template <typename T>
__global__ void __launch_bounds__(128)
pool_blocks_kernel(T* __restrict__ summary, const T* __restrict__ cache, const int* __restrict__ block_table,
                   const int* __restrict__ tok_req, const int* __restrict__ positions, const int* __restrict__ sum_slots,
                   int bt_stride, int G, int d, int dv, int page_size, int block, int num_pages, long long num_sum_slots,
                   int vec_ok) {
  __shared__ long long s_row[kPoolStaged];     // page * page_stride + position in the page, -1: not held
  const int t = blockIdx.x;
  const long long sl = sum_slots[t];       // inputs of the step
  const int r = tok_req[t], p = positions[t];
  pdl_wait();
  pdl_launch_dependents();
  if (sl < 0 || sl >= num_sum_slots || r < 0 || p + 1 < block) return;
  const size_t page_stride = (size_t)G * page_size * (d + dv);
  const size_t v_plane = (size_t)G * page_size * d;
  const int* bt = block_table + (size_t)r * bt_stride;
  T* dst = summary + (size_t)(sl / page_size) * page_stride;
  const int off = (int)(sl % page_size);
  const float inv = 1.0f / (float)block;
  const int first = p - block + 1;
  auto row_of = [&](int j) -> long long {     // where position j lies: its page's start, and its row within a head's rows
    const int page = bt[j / page_size];
    return (page < 0 || page >= num_pages) ? -1 : (long long)page * (long long)page_stride;   // never follow a table entry outside the pool
  };
  const bool staged = block <= kPoolStaged;
  if (staged) {
    for (int j = threadIdx.x; j < block; j += blockDim.x) s_row[j] = row_of(first + j);
    __syncthreads();
  }
  constexpr int VN = Vec16<T>::N;
  const int step = vec_ok ? VN : 1;
  for (int idx = threadIdx.x * step; idx < G * (d + dv); idx += blockDim.x * step) {
    const bool is_v = idx >= G * d;
    const int g = is_v ? (idx - G * d) / dv : idx / d;
    const int e = is_v ? (idx - G * d) % dv : idx % d;
    const int wd = is_v ? dv : d;
    const size_t plane = is_v ? v_plane : 0;
    const size_t head = plane + (size_t)g * page_size * wd + e;
    float acc[VN];
#pragma unroll
    for (int u = 0; u < VN; ++u) acc[u] = 0.f;
    // four positions' loads are requested together; the sums run in ascending order of position
    for (int j0 = 0; j0 < block; j0 += 4) {
      Vec16<T> v[4];
      T one[4];
      bool have[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int j = j0 + u;
        have[u] = false;
        if (j < block) {
          const long long base = staged ? s_row[j] : row_of(first + j);
          if (base >= 0) {
            const T* src = cache + base + head + (size_t)((first + j) % page_size) * wd;
            have[u] = true;
            if (vec_ok) v[u] = load16(src); else one[u] = *src;
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (have[u]) {
          if (vec_ok) {
#pragma unroll
            for (int x = 0; x < VN; ++x) acc[x] += v[u].get(x);
          } else {
            acc[0] += to_f32(one[u]);
          }
        }
      }
    }
    T* out = dst + head + (size_t)off * wd;
    if (vec_ok) {
      Vec16<T> o;
#pragma unroll
      for (int x = 0; x < VN; ++x) o.set(x, acc[x] * inv);
      store16(out, o);
    } else {
      *out = from_f32<T>(acc[0] * inv);
    }
  }
}

template <typename T>
int pool_blocks(void* summary, const void* cache, const int* block_table, const int* tok_req, const int* positions,
                const int* sum_slots, int tokens, int bt_stride, int G, int d, int dv, int page_size, int block, int num_pages,
                long long num_sum_slots, void* stream) {
  PTL_REQUIRE(tokens >= 0 && G > 0 && d > 0 && dv > 0 && page_size > 0 && block > 0 && num_pages > 0, "pool_blocks: bad sizes");
  if (tokens == 0) return 0;
  constexpr int VN = Vec16<T>::N;
  const int vec_ok = d % VN == 0 && dv % VN == 0 && aligned16(cache) && aligned16(summary);      // every row starts a packet
  return launch_kernel("pool_blocks", pool_blocks_kernel<T>, dim3(tokens), dim3(128), 0, as_stream(stream), (T*)summary,
                       (const T*)cache, block_table, tok_req, positions, sum_slots, bt_stride, G, d, dv, page_size, block,
                       num_pages, num_sum_slots, vec_ok);
}

// ------------------------------------------------------------------ attention
constexpr int kWaMaxPerLane = 16;  // value heads up to 512 (kernels are built for 8 and for 16 values per lane)
constexpr int kWaWarps = 4;

__device__ __forceinline__ void wa_two_fma(float& hi, float& lo, float a, float b) {
  const float h = __fmul_rn(a, b);
  const float r = fmaf(a, b, -h);
  const float t = __fadd_rn(hi, h);
  const float z = __fsub_rn(t, hi);
  const float e = __fadd_rn(__fsub_rn(hi, __fsub_rn(t, z)), __fsub_rn(h, z));
  hi = t;
  lo = __fadd_rn(lo, __fadd_rn(e, r));
}
__device__ __forceinline__ float2 unpack_pair(uint32_t v) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v));
}
__device__ __forceinline__ void wa_two_scale(float& hi, float& lo, float c) {
  const float h = __fmul_rn(hi, c);
  lo = fmaf(lo, c, fmaf(hi, c, -h));
  hi = h;
}

template <typename T, int MPL>
__global__ void __launch_bounds__(kWaWarps * 32)
window_attention_kernel(T* __restrict__ out, float* __restrict__ part_acc, float* __restrict__ part_ml,
                        const T* __restrict__ q, const T* __restrict__ cache, const int* __restrict__ block_table,
                        const int* __restrict__ tok_req, const int* __restrict__ positions, int q_stride, int out_stride,
                        int bt_stride, int H, int G, int d, int dv, int page_size, float scale, int window, int keep,
                        int splits, int num_pages, int vec_ok, const int* __restrict__ items, int wide_ok, int shared_v,
                        int sink, float temp_coef, int temp_every, float bias_exp, int gate_col, int pool,
                        const T* __restrict__ summary, const int* __restrict__ sum_bt, int sum_bt_stride, int sum_pages) {
  constexpr int kWaMaxPerLane = MPL;   // values of a head that a lane holds
  extern __shared__ float qs_all[];  // [warps][d]
  __shared__ float s_pr[kWaWarps][32];
  __shared__ unsigned long long s_vb[kWaWarps][32];
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = items ? items[blockIdx.x] : blockIdx.x;
  const int h = blockIdx.y * kWaWarps + warp;
  if (h >= H) return;
  const int split = blockIdx.z;
  float* qs = qs_all + warp * d;
  const T* qrow = q + (size_t)t * q_stride + (size_t)h * d;
  constexpr bool kCompensated = sizeof(T) == 4;
  const int r = tok_req[t];        // r < 0: a padding row; it sees no key and yields zeros
  const int p = positions[t];
  if (temp_coef != 0.f) scale *= fmaf(temp_coef, logf((float)((p + 1) / temp_every) + 1.0f), 1.0f);
  for (int i = lane; i < d; i += 32) qs[i] = kCompensated ? to_f32(qrow[i]) : to_f32(qrow[i]) * scale;
  __syncwarp();

  const int lo = (window > 0 && p - window + 1 > 0) ? p - window + 1 : 0;
  const int n_keep = min(keep, lo);                 // kept positions that the window has passed
  const int n_pool = (pool > 0 && window > 0 && r >= 0 && p - window + 1 > 0) ? (p - window + 1) / pool : 0;   // whole blocks behind the window
  const int n_pool_pad = (n_pool + 31) & ~31;
  const int n_list = r < 0 ? 0 : n_pool_pad + n_keep + (p - lo + 1);
  const float slope = bias_exp > 0.f ? exp2f(-bias_exp * (float)(h + 1) / (float)H) : 0.f;
  int chunk = (n_list + splits - 1) / splits;
  chunk = (chunk + 31) & ~31;
  const int i_begin = split * chunk;
  const int i_end = min(i_begin + chunk, n_list);
  const int g = h / (H / G);
  const size_t page_stride = (size_t)G * page_size * (d + (shared_v ? 0 : dv));
  const size_t v_plane = shared_v ? 0 : (size_t)G * page_size * d;
  const int v_row = shared_v ? d : dv;      // elements between the values of neighbouring keys
  const int* bt = block_table + (size_t)(r < 0 ? 0 : r) * bt_stride;
  const int* sbt = sum_bt ? sum_bt + (size_t)(r < 0 ? 0 : r) * sum_bt_stride : nullptr;
  constexpr int VN = Vec16<T>::N;

  float m = -INFINITY, l = 0.f, l_lo = 0.f;
  float acc[kWaMaxPerLane], acc_lo[kWaMaxPerLane];
#pragma unroll
  for (int i = 0; i < kWaMaxPerLane; ++i) { acc[i] = 0.f; acc_lo[i] = 0.f; }

  for (int i0 = i_begin; i0 < i_end; i0 += 32) {
    const int li = i0 + lane;
    bool valid = li < i_end;
    const bool mean = li < n_pool_pad;                  // the same for all lanes of a turn
    if (mean && li >= n_pool) valid = false;
    const int lt = li - n_pool_pad;
    const int key = mean ? li : (lt < n_keep ? lt : lo + (lt - n_keep));     // a block's number, or a position
    const T* vptr = cache + v_plane;
    float s = -INFINITY;
    const int page = valid ? (mean ? sbt[key / page_size] : bt[key / page_size]) : 0;
    if (page < 0 || page >= (mean ? sum_pages : num_pages)) valid = false;   // never follow a table entry outside the pool
    if (valid) {
      const size_t in_page = (size_t)g * page_size + key % page_size;
      const T* pg = (mean ? summary : cache) + (size_t)page * page_stride;
      const T* kp = pg + in_page * d;
      vptr = pg + v_plane + in_page * v_row;
      float dot = 0.f, dot_lo = 0.f;
      if (vec_ok) {
        // four packets of the key row are requested together and used afterwards: a product right behind its load
        // holds the warp for the load's whole latency, once per packet
        for (int i = 0; i < d; i += 4 * VN) {
          Vec16<T> kv[4];
#pragma unroll
          for (int u = 0; u < 4; ++u)
            if (i + u * VN < d) kv[u] = load16(kp + i + u * VN);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (i + u * VN < d) {
#pragma unroll
              for (int e = 0; e < VN; ++e) {
                if constexpr (kCompensated) wa_two_fma(dot, dot_lo, qs[i + u * VN + e], kv[u].get(e));
                else dot = fmaf(qs[i + u * VN + e], kv[u].get(e), dot);
              }
            }
          }
        }
      } else {
        for (int i = 0; i < d; ++i) {
          if constexpr (kCompensated) wa_two_fma(dot, dot_lo, qs[i], to_f32(kp[i]));
          else dot = fmaf(qs[i], to_f32(kp[i]), dot);
        }
      }
      s = kCompensated ? __fadd_rn(dot, dot_lo) * scale : dot;
      if (!mean) s = fmaf(-slope, (float)(p - key), s);
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float pr = valid ? expf(s - m_new) : 0.f;
    const float alpha = expf(m - m_new);
    if constexpr (kCompensated) {
      if (alpha != 1.f) {
        wa_two_scale(l, l_lo, alpha);
#pragma unroll
        for (int i = 0; i < kWaMaxPerLane; ++i) wa_two_scale(acc[i], acc_lo[i], alpha);
      }
      wa_two_fma(l, l_lo, warp_sum(pr), 1.f);
    } else {
      l = l * alpha + warp_sum(pr);
#pragma unroll
      for (int i = 0; i < kWaMaxPerLane; ++i) acc[i] *= alpha;
    }
    m = m_new;
    // every lane needs every key's weight and value row: they go through shared memory, so that the walk below has
    // neither shuffles nor branches and several keys' loads are in flight (a key that is not seen has weight 0 and the
    // address of the cache's first value row)
    __syncwarp();
    s_pr[warp][lane] = pr;
    s_vb[warp][lane] = (unsigned long long)vptr;
    __syncwarp();
    const int nvalid = min(32, i_end - i0);
    // (lanes past the list's end hold weight 0 and the address of a value row that exists, so the walks below take
    // whole batches of keys: their loads are requested together and used afterwards)
    if (wide_ok) {
      // value heads of 32 * CH elements, CH = 2 or 4: a lane owns CH neighbours and fetches them as one word or two
#pragma unroll
      for (int j0 = 0; j0 < 32; j0 += 8) {
        if (j0 >= nvalid) break;
        uint2 raw[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const T* vp = reinterpret_cast<const T*>(s_vb[warp][j0 + u]) + lane * wide_ok;
          if (wide_ok == 4) raw[u] = *reinterpret_cast<const uint2*>(vp);
          else raw[u].x = *reinterpret_cast<const uint32_t*>(vp);
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const float pj = s_pr[warp][j0 + u];
          const float2 a = unpack_pair(raw[u].x);
          acc[0] = fmaf(pj, a.x, acc[0]);
          acc[1] = fmaf(pj, a.y, acc[1]);
          if (wide_ok == 4) {
            const float2 b = unpack_pair(raw[u].y);
            acc[2] = fmaf(pj, b.x, acc[2]);
            acc[3] = fmaf(pj, b.y, acc[3]);
          }
        }
      }
    } else {
      for (int j0 = 0; j0 < nvalid; j0 += 4) {
        T raw[4][kWaMaxPerLane];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const T* vp = reinterpret_cast<const T*>(s_vb[warp][j0 + u]);
#pragma unroll
          for (int i = 0; i < kWaMaxPerLane; ++i) {
            const int dd = lane + 32 * i;
            if (dd < dv) raw[u][i] = vp[dd];
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float pj = s_pr[warp][j0 + u];
#pragma unroll
          for (int i = 0; i < kWaMaxPerLane; ++i) {
            const int dd = lane + 32 * i;
            if (dd < dv) {
              if constexpr (kCompensated) wa_two_fma(acc[i], acc_lo[i], pj, to_f32(raw[u][i]));
              else acc[i] = fmaf(pj, to_f32(raw[u][i]), acc[i]);
            }
          }
        }
      }
    }
  }
  if constexpr (kCompensated) {
    l = __fadd_rn(l, l_lo);
#pragma unroll
    for (int i = 0; i < kWaMaxPerLane; ++i) acc[i] = __fadd_rn(acc[i], acc_lo[i]);
  }
  if (splits == 1) {
    if (sink) {            // the term of score 0 joins as a key would: the maximum may move to 0, and exp(0 - maximum) is added
      const float m_all = fmaxf(m, 0.f);
      const float a = expf(m - m_all);
      l = fmaf(l, a, expf(-m_all));
#pragma unroll
      for (int i = 0; i < kWaMaxPerLane; ++i) acc[i] *= a;
    }
    const float inv = l > 0.f ? 1.0f / l : 0.f;
    T* o = out + (size_t)t * out_stride + (size_t)h * dv;
    const T* gate = gate_col >= 0 ? q + (size_t)t * q_stride + gate_col + (size_t)h * dv : nullptr;
#pragma unroll
    for (int i = 0; i < kWaMaxPerLane; ++i) {
      const int dd = wide_ok ? lane * wide_ok + i : lane + 32 * i;
      if (dd < dv && (!wide_ok || i < wide_ok)) {
        float res = acc[i] * inv;
        if (gate) res *= 1.0f / (1.0f + expf(-to_f32(gate[dd])));
        o[dd] = from_f32<T>(res);
      }
    }
  } else {
    const size_t idx = ((size_t)t * H + h) * splits + split;
    float* pa = part_acc + idx * dv;
#pragma unroll
    for (int i = 0; i < kWaMaxPerLane; ++i) {
      const int dd = wide_ok ? lane * wide_ok + i : lane + 32 * i;
      if (dd < dv && (!wide_ok || i < wide_ok)) pa[dd] = acc[i];
    }
    if (lane == 0) { part_ml[idx * 2] = m; part_ml[idx * 2 + 1] = l; }
  }
}

// out = sum_z e^{m_z - M} acc_z / sum_z e^{m_z - M} l_z over the parts of the key list, in the order of the parts.
template <typename T, int MPL>
__global__ void __launch_bounds__(kWaWarps * 32)
window_attention_merge_kernel(T* __restrict__ out, const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                              int out_stride, int H, int dv, int splits, int tokens, const int* __restrict__ items, int sink,
                              const T* __restrict__ q, int q_stride, int gate_col) {
  constexpr int kWaMaxPerLane = MPL;
  pdl_wait();
  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long pair = (long long)blockIdx.x * kWaWarps + warp;
  if (pair >= (long long)tokens * H) return;
  const int t = items ? items[pair / H] : (int)(pair / H);
  const int h = (int)(pair % H);
  const size_t idx0 = ((size_t)t * H + h) * splits;
  // lane z holds the (maximum, sum) of part z, 32 parts at a time; the weights are handed round by shuffles and the
  // parts' accumulators are fetched four at a time
  float M = -INFINITY;
  for (int z = lane; z < splits; z += 32) M = fmaxf(M, part_ml[(idx0 + z) * 2]);
  M = warp_max(M);
  if (sink) M = fmaxf(M, 0.f);
  float L = 0.f;
  float acc[kWaMaxPerLane];
#pragma unroll
  for (int i = 0; i < kWaMaxPerLane; ++i) acc[i] = 0.f;
  for (int z0 = 0; z0 < splits; z0 += 32) {
    const int z = z0 + lane;
    float wz = 0.f;
    if (z < splits) {
      const float mz = part_ml[(idx0 + z) * 2];
      if (mz > -INFINITY) {
        wz = expf(mz - M);
        L = fmaf(wz, part_ml[(idx0 + z) * 2 + 1], L);
      }
    }
    const int n = min(32, splits - z0);
    for (int j0 = 0; j0 < n; j0 += 4) {
      float raw[4][kWaMaxPerLane];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float* pa = part_acc + (idx0 + z0 + min(j0 + u, n - 1)) * dv;     // an empty part wrote zeros
#pragma unroll
        for (int i = 0; i < kWaMaxPerLane; ++i) {
          const int dd = lane + 32 * i;
          if (dd < dv) raw[u][i] = pa[dd];
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float wj = __shfl_sync(0xffffffffu, wz, min(j0 + u, 31));
        if (j0 + u < n) {
#pragma unroll
          for (int i = 0; i < kWaMaxPerLane; ++i) {
            const int dd = lane + 32 * i;
            if (dd < dv) acc[i] = fmaf(wj, raw[u][i], acc[i]);
          }
        }
      }
    }
  }
  L = warp_sum(L);
  if (sink) L += expf(-M);
  const float inv = L > 0.f ? 1.0f / L : 0.f;
  T* o = out + (size_t)t * out_stride + (size_t)h * dv;
  const T* gate = gate_col >= 0 ? q + (size_t)t * q_stride + gate_col + (size_t)h * dv : nullptr;
#pragma unroll
  for (int i = 0; i < kWaMaxPerLane; ++i) {
    const int dd = lane + 32 * i;
    if (dd < dv) {
      float res = acc[i] * inv;
      if (gate) res *= 1.0f / (1.0f + expf(-to_f32(gate[dd])));
      o[dd] = from_f32<T>(res);
    }
  }
}

template <typename T>
int window_attention(void* out, const void* q, const void* cache, const int* block_table, const int* tok_req,
                     const int* positions, float* part_acc, float* part_ml, int tokens, int q_stride, int out_stride,
                     int bt_stride, int H, int G, int d, int dv, int page_size, float scale, int window, int keep, int splits,
                     int num_pages, const int* items, int shared_v, int sink, float temp_coef, int temp_every, float bias_exp,
                     int gate_col, int pool, const void* summary, const int* sum_bt, int sum_bt_stride, int sum_pages,
                     void* stream) {
  PTL_REQUIRE(tokens >= 0 && H > 0 && G > 0 && page_size > 0 && d > 0, "window_attention: bad sizes");
  PTL_REQUIRE(pool == 0 || (summary && sum_bt && sum_pages > 0 && window > 0 && keep == 0 && !shared_v && !sink),
              "window_attention: means of blocks need their pages and a window, and go with no kept positions, shared values or sink");
  PTL_REQUIRE(bias_exp >= 0.f && (gate_col < 0 || gate_col + H * dv <= q_stride), "window_attention: bad bias or gate column");
  PTL_REQUIRE(!shared_v || dv <= d, "window_attention: values of %d entries inside keys of %d", dv, d);
  PTL_REQUIRE(temp_every >= 1, "window_attention: temp_every=%d", temp_every);
  PTL_REQUIRE(H % G == 0, "window_attention: %d query heads are no multiple of %d kv heads", H, G);
  PTL_REQUIRE(dv >= 1 && dv <= 32 * kWaMaxPerLane, "window_attention: value heads of %d, at most %d", dv, 32 * kWaMaxPerLane);
  PTL_REQUIRE(d <= 2048, "window_attention: head size %d", d);
  PTL_REQUIRE(splits >= 1 && splits <= 65535, "window_attention: splits=%d", splits);
  PTL_REQUIRE(splits == 1 || (part_acc && part_ml), "window_attention: splits > 1 need scratch buffers");
  PTL_REQUIRE(window >= 0 && keep >= 0 && num_pages > 0, "window_attention: window and kept positions must be >= 0");
  if (tokens == 0) return 0;
  constexpr int VN = Vec16<T>::N;
  const int dv_stored = shared_v ? 0 : dv;
  const int vec_ok = aligned16(cache) && d % VN == 0 && ((size_t)page_size * G * (d + dv_stored)) % VN == 0 &&
                     ((size_t)G * page_size * d) % VN == 0;
  // bfloat16 value heads of 64 or 128 whose rows start on 8-byte boundaries: a lane fetches 2 or 4 neighbours at once
  int wide_ok = 0;
  if (sizeof(T) == 2 && (dv == 64 || dv == 128) && aligned16(cache) && ((size_t)G * page_size * d) % 4 == 0 &&
      ((size_t)page_size * G * (d + dv_stored)) % 4 == 0 && (!shared_v || d % 4 == 0))
    wide_ok = dv / 32;
  dim3 grid(tokens, (H + kWaWarps - 1) / kWaWarps, splits);
  const size_t smem = (size_t)kWaWarps * d * sizeof(float);
  const long long pairs = (long long)tokens * H;
#define PTL_WA_LAUNCH(MPL)                                                                                                         \
  {                                                                                                                                \
    int rc = launch_kernel("window_attention", window_attention_kernel<T, MPL>, grid, dim3(kWaWarps * 32), smem,                   \
                           as_stream(stream), (T*)out, part_acc, part_ml, (const T*)q, (const T*)cache, block_table, tok_req,      \
                           positions, q_stride, out_stride, bt_stride, H, G, d, dv, page_size, scale, window, keep, splits,        \
                           num_pages, vec_ok, items, wide_ok, shared_v, sink, temp_coef, temp_every, bias_exp, gate_col, pool,     \
                           (const T*)summary, sum_bt, sum_bt_stride, sum_pages);                                                  \
    if (rc || splits <= 1) return rc;                                                                                              \
    return launch_kernel("window_attention_merge", window_attention_merge_kernel<T, MPL>,                                          \
                         dim3((unsigned)((pairs + kWaWarps - 1) / kWaWarps)), dim3(kWaWarps * 32), 0, as_stream(stream), (T*)out,  \
                         (const float*)part_acc, (const float*)part_ml, out_stride, H, dv, splits, tokens, items, sink,            \
                         (const T*)q, q_stride, gate_col);                                                                         \
  }
  if (dv <= 32 * 8) PTL_WA_LAUNCH(8)      // (value heads up to 256 keep the registers of 8 values per lane)
  PTL_WA_LAUNCH(16)
#undef PTL_WA_LAUNCH
}

}  // namespace ptl

#define PTL_WINDOW_ATTENTION(SUFFIX, TYPE)                                                                                         \
  PTL_EXPORT int ptl_qk_norm_rotate_store##SUFFIX(void* proj, int tokens, int ld, int H, int G, int d, int dv, const float* wq,     \
                                                  const float* wk, float eps, const int* positions, const float* freq, int dims,   \
                                                  float amplitude, const int* slots, void* cache, int page_size,                   \
                                                  long long num_slots, void* stream) {                                             \
    return ptl::qk_norm_rotate_store<TYPE>(proj, tokens, ld, H, G, d, dv, wq, wk, eps, positions, freq, dims, amplitude, slots,     \
                                           cache, page_size, num_slots, stream);                                                   \
  }                                                                                                                                \
  PTL_EXPORT int ptl_window_attention##SUFFIX(void* out, const void* q, const void* cache, const int* block_table,                  \
                                              const int* tok_req, const int* positions, float* part_acc, float* part_ml,           \
                                              int tokens, int q_stride, int out_stride, int bt_stride, int H, int G, int d, int dv, \
                                              int page_size, float scale, int window, int keep, int splits, int num_pages,         \
                                              const int* items, int shared_v, int sink, float temp_coef, int temp_every,           \
                                              float bias_exp, int gate_col, int pool, const void* summary, const int* sum_bt,      \
                                              int sum_bt_stride, int sum_pages, void* stream) {                                    \
    return ptl::window_attention<TYPE>(out, q, cache, block_table, tok_req, positions, part_acc, part_ml, tokens, q_stride,        \
                                       out_stride, bt_stride, H, G, d, dv, page_size, scale, window, keep, splits, num_pages,      \
                                       items, shared_v, sink, temp_coef, temp_every, bias_exp, gate_col, pool, summary, sum_bt,    \
                                       sum_bt_stride, sum_pages, stream);                                                          \
  }                                                                                                                                \
  PTL_EXPORT int ptl_head_norm_rotate_store##SUFFIX(void* proj, int tokens, int ld, int H, int G, int d, int dv, const float* wq,   \
                                                    const float* wk, float eps, const int* positions, const void* inv_freq,        \
                                                    int freq64, int rot, const int* slots, void* cache, int page_size,             \
                                                    long long num_slots, void* stream) {                                           \
    return ptl::head_norm_rotate_store<TYPE>(proj, tokens, ld, H, G, d, dv, wq, wk, eps, positions, inv_freq, freq64, rot, slots,   \
                                             cache, page_size, num_slots, stream);                                                 \
  }                                                                                                                                \
  PTL_EXPORT int ptl_pool_blocks##SUFFIX(void* summary, const void* cache, const int* block_table, const int* tok_req,              \
                                         const int* positions, const int* sum_slots, int tokens, int bt_stride, int G, int d,      \
                                         int dv, int page_size, int block, int num_pages, long long num_sum_slots, void* stream) { \
    return ptl::pool_blocks<TYPE>(summary, cache, block_table, tok_req, positions, sum_slots, tokens, bt_stride, G, d, dv,          \
                                  page_size, block, num_pages, num_sum_slots, stream);                                             \
  }
PTL_WINDOW_ATTENTION(_f32, float)
PTL_WINDOW_ATTENTION(_bf16, __nv_bfloat16)
