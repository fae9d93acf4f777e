// Generalized delta rule: per head a float32 state S [d, d] (rows: key channels, columns: value channels),
//   S <- diag(w_t) S - (a_t * u_t) (u_t^T S) + k_t v_t^T,   o_t = S^T r_t,   u_t = k_t / sqrt(|k_t|^2 + unit_eps),
// both products on the right reading the old S, with per key channel
//   w_t = exp(-decay_limit * sigmoid(z_t + w_bias)),   a_t = sigmoid(a_pre_t + a_bias).
//
// proj is the projection's output [T, r | k | v | ...] (H heads of d each), a_pre the first H*d columns of a float32
// array with rows of a_ld floats, z float32 [T, H*d] (the decay's argument before its bias, made by
// lowrank_tanh_linear below).  The layout of the walk is that of the gated delta rule (recurrent.cu): eight lanes
// share a column of the state, lane l holding the row pairs (16 m + 2 l, 16 m + 2 l + 1) as float2; a block of 128
// threads walks 16 columns of one head of one request through its tokens in order.  Tokens come in batches of
// kGdBatch: all threads bring a batch's r and k of the head, its decays, removal rates and 16 values into shared
// memory (sigmoids and exponentials worked out while staging; the next batch's inputs are held in registers while
// this one is walked).  With c = -(u^T S) / sqrt(|k|^2 + unit_eps) per column, a row's update is
//   S <- w S + (a k) c + k v,
// three two-wide fused multiply-adds per row pair.  Everything after the loads is float32; a token's result does
// not depend on how the request was cut into steps or on what else the step holds.  The state of a request is read
// from its slot unless the portion starts at position 0, and written back at the end.
#include "common.cuh"

namespace ptl {

constexpr int kGdBatch = 16;

__device__ __forceinline__ float sigmoid_f32(float x) { return 1.0f / (1.0f + expf(-x)); }

template <typename T, int RPL>
__global__ void __launch_bounds__(128)
general_delta_kernel(float* __restrict__ out, const T* __restrict__ proj, int ld, const float* __restrict__ a_pre, int a_ld,
                     const float* __restrict__ a_bias, const float* __restrict__ z, const float* __restrict__ w_bias,
                     float decay_limit, float* __restrict__ state, const int* __restrict__ q_start,
                     const int* __restrict__ positions, const int* __restrict__ state_slot, int heads, int d, float unit_eps) {
  static_assert(RPL % 2 == 0, "a lane holds pairs of rows");
  constexpr int DS = 8 * RPL;                       // floats between tokens' rows in shared memory
  constexpr int HP = RPL / 2;                       // row pairs of a lane
  extern __shared__ __align__(16) float gd_smem[];
  float* s_r = gd_smem;                            // [batch][DS]
  float* s_k = s_r + kGdBatch * DS;
  float* s_w = s_k + kGdBatch * DS;                // decay per row
  float* s_ak = s_w + kGdBatch * DS;               // removal rate times key per row
  float* s_v = s_ak + kGdBatch * DS;               // [batch][16]
  float* s_kn = s_v + kGdBatch * 16;               // 1 / (|k|^2 + unit_eps) per token
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.z, h = blockIdx.y;
  const int lo = q_start[r], hi = q_start[r + 1];
  if (hi <= lo || state_slot[r] < 0) return;
  const int sub = threadIdx.x & 7, grp = threadIdx.x >> 3;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int j0 = blockIdx.x * 16;
  const bool live = j0 + grp < d;
  const int j = live ? j0 + grp : d - 1;
  const int n = heads * d;
  float* st = state + (((size_t)state_slot[r] * heads + h) * d) * d + j;
  const bool from_zero = positions[lo] == 0;
  float2 S[HP];
#pragma unroll
  for (int m = 0; m < HP; ++m) {
    const int row = 16 * m + 2 * sub;
    S[m].x = (row < d && !from_zero) ? st[(size_t)row * d] : 0.f;
    S[m].y = (row + 1 < d && !from_zero) ? st[(size_t)(row + 1) * d] : 0.f;
  }
  for (int i = threadIdx.x; i < 4 * kGdBatch * DS; i += blockDim.x) s_r[i] = 0.f;   // (s_k, s_w, s_ak follow s_r) zero beyond d for good
  // Element i of a thread's share of a batch: flat index threadIdx.x + 128 * i over [batch][d]; RPL of them cover
  // kGdBatch * d = 16 d <= 128 * RPL (d <= 8 * RPL).  They are kept as fetched and converted when they go to shared
  // memory, after the walk over the batch before: the loads are in flight during that walk.
  T pr[RPL], pk[RPL], pv[2];
  float pz[RPL], pa[RPL];
  const int tok_first = threadIdx.x / d, e_first = threadIdx.x % d, tok_step = 128 / d, e_step = 128 % d;
  auto fetch = [&](int t0) {
    const int nb = min(kGdBatch, hi - t0);
    int tok = tok_first, e = e_first;
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
      if (tok < nb) {
        const size_t t = (size_t)(t0 + tok);
        pr[i] = proj[t * ld + h * d + e];
        pk[i] = proj[t * ld + n + h * d + e];
        pz[i] = z[t * n + h * d + e];
        pa[i] = a_pre[t * a_ld + h * d + e];
      }
      tok += tok_step;
      e += e_step;
      if (e >= d) { e -= d; ++tok; }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = threadIdx.x + 128 * i;
      if ((idx >> 4) < nb) pv[i] = proj[(size_t)(t0 + (idx >> 4)) * ld + 2 * n + h * d + min(j0 + (idx & 15), d - 1)];
    }
  };
  fetch(lo);
  for (int t0 = lo; t0 < hi; t0 += kGdBatch) {
    const int nb = min(kGdBatch, hi - t0);
    __syncthreads();                                  // the batch before has been walked (and the rows are zeroed)
    {
      int tok = tok_first, e = e_first;
#pragma unroll
      for (int i = 0; i < RPL; ++i) {
        if (tok < nb) {
          const float kf = to_f32(pk[i]);
          s_r[tok * DS + e] = to_f32(pr[i]);
          s_k[tok * DS + e] = kf;
          s_w[tok * DS + e] = expf(-decay_limit * sigmoid_f32(pz[i] + w_bias[h * d + e]));
          s_ak[tok * DS + e] = sigmoid_f32(pa[i] + a_bias[h * d + e]) * kf;
        }
        tok += tok_step;
        e += e_step;
        if (e >= d) { e -= d; ++tok; }
      }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = threadIdx.x + 128 * i;
      if ((idx >> 4) < nb) s_v[idx] = to_f32(pv[i]);
    }
    __syncthreads();
    if (t0 + kGdBatch < hi) fetch(t0 + kGdBatch);     // in flight while this batch is walked
    {
      // the squared lengths of the keys: warp w takes tokens w, w + 4, w + 8, w + 12
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const int tok = warp + 4 * m;
        if (tok < nb) {
          float kk = 0.f;
          for (int e = lane; e < d; e += 32) kk = fmaf(s_k[tok * DS + e], s_k[tok * DS + e], kk);
          kk = warp_sum(kk);
          if (lane == 0) s_kn[tok] = 1.0f / (kk + unit_eps);
        }
      }
    }
    __syncthreads();
#pragma unroll (RPL <= 16 ? 2 : 1)
    for (int tok = 0; tok < nb; ++tok) {
      const float2* kp = reinterpret_cast<const float2*>(s_k + tok * DS) + sub;     // pair m of this lane: kp[8 * m]
      const float2* rp = reinterpret_cast<const float2*>(s_r + tok * DS) + sub;
      const float2* wp = reinterpret_cast<const float2*>(s_w + tok * DS) + sub;
      const float2* ap = reinterpret_cast<const float2*>(s_ak + tok * DS) + sub;
      float2 k[HP];
      float2 dot0 = make_float2(0.f, 0.f), dot1 = make_float2(0.f, 0.f);
#pragma unroll
      for (int m = 0; m < HP; ++m) {
        k[m] = kp[8 * m];
        if (m & 1) dot1 = __ffma2_rn(S[m], k[m], dot1); else dot0 = __ffma2_rn(S[m], k[m], dot0);
      }
      float dot = (dot0.x + dot0.y) + (dot1.x + dot1.y);
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float c = -dot * s_kn[tok];
      const float v = s_v[tok * 16 + grp];
      const float2 c2 = make_float2(c, c), v2 = make_float2(v, v);
      float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
      for (int m = 0; m < HP; ++m) {
        S[m] = __ffma2_rn(wp[8 * m], S[m], __ffma2_rn(ap[8 * m], c2, __fmul2_rn(k[m], v2)));
        const float2 rv = rp[8 * m];
        if (m & 1) acc1 = __ffma2_rn(S[m], rv, acc1); else acc0 = __ffma2_rn(S[m], rv, acc0);
      }
      float acc = (acc0.x + acc0.y) + (acc1.x + acc1.y);
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (sub == 0 && live) out[(size_t)(t0 + tok) * n + h * d + j] = acc;
    }
  }
  if (live) {
#pragma unroll
    for (int m = 0; m < HP; ++m) {
      const int row = 16 * m + 2 * sub;
      if (row < d) st[(size_t)row * d] = S[m].x;
      if (row + 1 < d) st[(size_t)(row + 1) * d] = S[m].y;
    }
  }
}

template <typename T>
int general_delta_scan(float* out, const void* proj, int ld, const float* a_pre, int a_ld, const float* a_bias, const float* z,
                       const float* w_bias, float decay_limit, float* state, const int* q_start, const int* positions,
                       const int* state_slot, int requests, int heads, int d, float unit_eps, void* stream) {
  PTL_REQUIRE(requests >= 0 && heads > 0 && d > 0 && d <= 256, "general_delta_scan: bad sizes heads=%d d=%d (at most 256)", heads, d);
  PTL_REQUIRE(ld >= 3 * heads * d && a_ld >= heads * d, "general_delta_scan: rows are too short");
  PTL_REQUIRE(requests <= 65535 && heads <= 65535, "general_delta_scan: at most 65535 requests and heads");
  if (requests == 0) return 0;
  const dim3 grid((d + 15) / 16, heads, requests), block(128);
  static SmemRaised raised[6];
#define PTL_GD(RPL, SLOT)                                                                                                      \
  {                                                                                                                            \
    const size_t smem = (size_t)kGdBatch * (4 * 8 * RPL + 16 + 1) * sizeof(float);                                             \
    if (smem > 48 * 1024)                                                                                                      \
      if (int rc = raise_shared_memory("general_delta_scan", general_delta_kernel<T, RPL>, (int)smem, raised[SLOT])) return rc; \
    return launch_kernel("general_delta_scan", general_delta_kernel<T, RPL>, grid, block, smem, as_stream(stream), out,        \
                         (const T*)proj, ld, a_pre, a_ld, a_bias, z, w_bias, decay_limit, state, q_start, positions,           \
                         state_slot, heads, d, unit_eps);                                                                      \
  }
  const int per_lane = (d + 7) / 8;
  if (per_lane <= 2) PTL_GD(2, 0)
  if (per_lane <= 4) PTL_GD(4, 1)
  if (per_lane <= 8) PTL_GD(8, 2)
  if (per_lane <= 12) PTL_GD(12, 3)
  if (per_lane <= 16) PTL_GD(16, 4)
  PTL_GD(32, 5)
#undef PTL_GD
}

// z[t, c] = sum_j w2[c, j] * tanh(x[t, column + j]), float32 throughout.  Every result is one chain of fused
// multiply-adds, j ascending, whatever the tile it falls into, so a token's row has the same bits in a prompt
// portion and alone.  A block takes kLtTokens tokens and kLtCols columns: the inner inputs' tanh and a slab of w2
// (kLtRank values of j at a time, transposed so that neighbouring threads read neighbouring words) go through shared
// memory; a thread holds one column's sums for all the block's tokens.
constexpr int kLtTokens = 16, kLtCols = 128, kLtRank = 32;

__global__ void __launch_bounds__(kLtCols)
lowrank_tanh_linear_kernel(float* __restrict__ z, const float* __restrict__ x, int tokens, int x_ld, int column, int rank,
                           const float* __restrict__ w2, int n) {
  __shared__ __align__(16) float s_hid[kLtRank][kLtTokens];      // tanh of the inner inputs, tokens side by side
  __shared__ float s_w[kLtRank][kLtCols + 1];
  pdl_wait();
  pdl_launch_dependents();
  const int t0 = blockIdx.y * kLtTokens, c0 = blockIdx.x * kLtCols;
  const int c = c0 + threadIdx.x;
  float acc[kLtTokens];
#pragma unroll
  for (int t = 0; t < kLtTokens; ++t) acc[t] = 0.f;
  for (int j0 = 0; j0 < rank; j0 += kLtRank) {
    const int nj = min(kLtRank, rank - j0);
    __syncthreads();                                               // the slab before has been used
    for (int e = threadIdx.x; e < kLtTokens * kLtRank; e += kLtCols) {
      const int t = e / kLtRank, jj = e % kLtRank;
      s_hid[jj][t] = (t0 + t < tokens && jj < nj) ? tanhf(x[(size_t)(t0 + t) * x_ld + column + j0 + jj]) : 0.f;
    }
    for (int e = threadIdx.x; e < kLtCols * kLtRank; e += kLtCols) {
      const int cc = e / kLtRank, jj = e % kLtRank;
      s_w[jj][cc] = (c0 + cc < n && jj < nj) ? w2[(size_t)(c0 + cc) * rank + j0 + jj] : 0.f;
    }
    __syncthreads();
    for (int jj = 0; jj < nj; ++jj) {
      const float w = s_w[jj][threadIdx.x];
      const float4* hp = reinterpret_cast<const float4*>(s_hid[jj]);
#pragma unroll
      for (int q = 0; q < kLtTokens / 4; ++q) {
        const float4 hv = hp[q];
        acc[4 * q + 0] = fmaf(w, hv.x, acc[4 * q + 0]);
        acc[4 * q + 1] = fmaf(w, hv.y, acc[4 * q + 1]);
        acc[4 * q + 2] = fmaf(w, hv.z, acc[4 * q + 2]);
        acc[4 * q + 3] = fmaf(w, hv.w, acc[4 * q + 3]);
      }
    }
  }
  if (c < n) {
#pragma unroll
    for (int t = 0; t < kLtTokens; ++t)
      if (t0 + t < tokens) z[(size_t)(t0 + t) * n + c] = acc[t];
  }
}

}  // namespace ptl

PTL_EXPORT int ptl_lowrank_tanh_linear(float* z, const float* x, int tokens, int x_ld, int column, int rank, const float* w2, int n,
                                       void* stream) {
  PTL_REQUIRE(tokens >= 0 && rank > 0 && n > 0 && column >= 0 && column + rank <= x_ld,
              "lowrank_tanh_linear: bad sizes rank=%d n=%d column=%d ld=%d", rank, n, column, x_ld);
  if (tokens == 0) return 0;
  const dim3 grid((n + ptl::kLtCols - 1) / ptl::kLtCols, (tokens + ptl::kLtTokens - 1) / ptl::kLtTokens);
  PTL_REQUIRE(grid.y <= 65535, "lowrank_tanh_linear: %d tokens in one call", tokens);
  return ptl::launch_kernel("lowrank_tanh_linear", ptl::lowrank_tanh_linear_kernel, grid, dim3(ptl::kLtCols), 0,
                            ptl::as_stream(stream), z, x, tokens, x_ld, column, rank, w2, n);
}

#define PTL_GENERAL_DELTA(SUFFIX, TYPE)                                                                                          \
  PTL_EXPORT int ptl_general_delta_scan##SUFFIX(float* out, const void* proj, int ld, const float* a_pre, int a_ld,               \
                                                const float* a_bias, const float* z, const float* w_bias, float decay_limit,     \
                                                float* state, const int* q_start, const int* positions, const int* state_slot,   \
                                                int requests, int heads, int d, float unit_eps, void* stream) {                  \
    return ptl::general_delta_scan<TYPE>(out, proj, ld, a_pre, a_ld, a_bias, z, w_bias, decay_limit, state, q_start, positions,   \
                                         state_slot, requests, heads, d, unit_eps, stream);                                      \
  }
PTL_GENERAL_DELTA(_f32, float)
PTL_GENERAL_DELTA(_bf16, __nv_bfloat16)
