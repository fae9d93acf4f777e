// Kernels of the mixers that carry a per-request state of fixed size from step to step: the short
// causal convolution, the selective scan, the gated delta rule, and the per-head norm with an output
// gate.  States are float32 arrays [slots, ...]; a request's slot is state_slot[r] (negative: a padding
// row of a captured step, skipped), and a request whose first token of the step has position 0 starts
// from zeros whatever its slot holds.  A step's
// tokens lie request after request: request r owns rows q_start[r] .. q_start[r + 1] - 1.
// T is the element type of the projections' results; everything inside is float32.
#include "common.cuh"

namespace ptl {

__device__ __forceinline__ float softplus_f32(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float silu_f32(float x) { return x / (1.0f + expf(-x)); }

// ------------------------------------------------------------------ causal convolution per channel
// y[t, c] = act(b[c] + sum_k w[c, k] * in[t - (taps - 1) + k, c]), `in` being the request's inputs: rows of
// this step, before them the taps - 1 inputs kept in the state, zeros before position 0.
// state[slot, j, c], j = 0 .. taps - 2, oldest first.  Reads the state only; conv_state_kernel moves it on.
template <typename T>
__global__ void causal_conv_kernel(T* __restrict__ out, const T* __restrict__ x, int ld, int column, int channels,
                                   const float* __restrict__ w, const float* __restrict__ b, int taps,
                                   const float* __restrict__ state, const int* __restrict__ q_start,
                                   const int* __restrict__ tok_req, const int* __restrict__ positions,
                                   const int* __restrict__ state_slot, int silu, float* __restrict__ state_out) {
  pdl_wait();
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int r = tok_req[t];
  if (r < 0) return;
  const int in_step = t - q_start[r];                 // rows of this request before t in this step
  const int pos = positions[t];
  const float* st = state + (size_t)state_slot[r] * (taps > 1 ? taps - 1 : 1) * channels;
  float acc = b ? b[c] : 0.f;
  if (state_out) {
    // every request brings one token: this thread is the only one that touches its channel of the request's state, so
    // it also moves the state on (entry j takes entry j + 1, the last one the token's input)
    float* so = state_out + (size_t)state_slot[r] * (taps - 1) * channels;
    const T x_raw = x[(size_t)t * ld + column + c];
    constexpr int kHeld = 7;                          // up to 8 taps: the entries are all read before any is written
    if (taps - 1 <= kHeld) {
      float v[kHeld], wt[kHeld];
#pragma unroll
      for (int j = 0; j < kHeld; ++j) {
        const bool there = j < taps - 1;
        v[j] = (there && pos - (taps - 1 - j) >= 0) ? st[(size_t)j * channels + c] : 0.f;
        wt[j] = there ? w[(size_t)c * taps + j] : 0.f;
      }
      const float x_now = to_f32(x_raw);
#pragma unroll
      for (int j = 0; j < kHeld; ++j) {
        if (j < taps - 1) {
          acc = fmaf(wt[j], v[j], acc);
          if (j > 0) so[(size_t)(j - 1) * channels + c] = v[j];
        }
      }
      acc = fmaf(w[(size_t)c * taps + taps - 1], x_now, acc);
      so[(size_t)(taps - 2) * channels + c] = x_now;
      out[(size_t)t * channels + c] = from_f32<T>(silu ? silu_f32(acc) : acc);
      return;
    }
    const float x_now = to_f32(x_raw);
    for (int j = 0; j < taps - 1; ++j) {
      const float v = pos - (taps - 1 - j) >= 0 ? st[(size_t)j * channels + c] : 0.f;
      acc = fmaf(w[(size_t)c * taps + j], v, acc);
      if (j > 0) so[(size_t)(j - 1) * channels + c] = v;
    }
    acc = fmaf(w[(size_t)c * taps + taps - 1], x_now, acc);
    so[(size_t)(taps - 2) * channels + c] = x_now;
    out[(size_t)t * channels + c] = from_f32<T>(silu ? silu_f32(acc) : acc);
    return;
  }
  for (int k = 0; k < taps; ++k) {
    const int back = taps - 1 - k;
    float v = 0.f;
    if (back <= in_step) v = to_f32(x[(size_t)(t - back) * ld + column + c]);
    else if (back <= pos) v = st[(size_t)(taps - 1 - (back - in_step)) * channels + c];
    acc = fmaf(w[(size_t)c * taps + k], v, acc);
  }
  out[(size_t)t * channels + c] = from_f32<T>(silu ? silu_f32(acc) : acc);
}

// The state after the step: the last taps - 1 inputs of each request.  New entry j takes the step's row
// n - (taps - 1) + j, or, where that lies before the step, the old entry j + n (zero before position 0).
// Ascending j reads only entries that have not been rewritten yet.
template <typename T>
__global__ void conv_state_kernel(float* __restrict__ state, const T* __restrict__ x, int ld, int column, int channels, int taps,
                                  const int* __restrict__ q_start, const int* __restrict__ positions,
                                  const int* __restrict__ state_slot) {
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int lo = q_start[r], n = q_start[r + 1] - lo;
  if (n <= 0 || state_slot[r] < 0) return;
  const int pos0 = positions[lo];
  float* st = state + (size_t)state_slot[r] * (taps - 1) * channels;
  for (int j = 0; j < taps - 1; ++j) {
    const int row = n - (taps - 1) + j;
    float v;
    if (row >= 0) v = to_f32(x[(size_t)(lo + row) * ld + column + c]);
    else v = pos0 + row >= 0 ? st[(size_t)(j + n) * channels + c] : 0.f;
    st[(size_t)j * channels + c] = v;
  }
}

// ------------------------------------------------------------------ selective scan
// Per channel c and state n:  S <- exp(dt A[c, n]) S + dt x B_n;  y = sum_n S C_n + D x;  out = y * silu(z),
// dt = softplus(dt_raw[t, c] + dt_bias[c]).  Eight lanes share a channel, lane l holding states l, l + 8, ...
// (NPL of them); a block of 128 threads walks 16 channels of one request through its tokens in order.
// The tokens come in batches of `tb`: the block first brings a batch's B | C rows, its 16 channels' x, step sizes
// (softplus applied) and gates (silu applied) into shared memory with all threads, so that the walk, whose steps
// depend on one another, waits for shared memory only; the batch's results leave the same way.
// Shared memory: tb * (2 * n_state + 64) floats.
template <typename T, int NPL>
__global__ void __launch_bounds__(128)
selective_scan_kernel(T* __restrict__ out, const T* __restrict__ xc, const float* __restrict__ dt_raw,
                      const float* __restrict__ dt_bias, const float* __restrict__ A, const T* __restrict__ bc,
                      const float* __restrict__ D, const T* __restrict__ z, int z_ld, int z_column, int inner, int n_state,
                      float* __restrict__ state, const int* __restrict__ q_start, const int* __restrict__ positions,
                      const int* __restrict__ state_slot, int tb) {
  extern __shared__ __align__(16) float scan_smem[];
  float* s_bc = scan_smem;                        // [tb][2 * n_state]
  float* s_x = s_bc + (size_t)tb * 2 * n_state;   // [tb][16]
  float* s_dt = s_x + tb * 16;
  float* s_gate = s_dt + tb * 16;
  float* s_y = s_gate + tb * 16;
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.y;
  const int lo = q_start[r], hi = q_start[r + 1];
  if (hi <= lo || state_slot[r] < 0) return;
  const int sub = threadIdx.x & 7, grp = threadIdx.x >> 3;
  const int c0 = blockIdx.x * 16;
  const bool live = c0 + grp < inner;
  const int c = live ? c0 + grp : inner - 1;          // lanes past the end shadow the last channel and store nothing
  float* st = state + ((size_t)state_slot[r] * inner + c) * n_state;
  const bool from_zero = positions[lo] == 0;
  float S[NPL], a[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int n = sub + 8 * i;
    S[i] = (n < n_state && !from_zero) ? st[n] : 0.f;
    a[i] = n < n_state ? A[(size_t)c * n_state + n] : 0.f;
  }
  const float skip = D[c];
  for (int t0 = lo; t0 < hi; t0 += tb) {
    const int nb = min(tb, hi - t0);
    __syncthreads();                                  // the batch before has been walked and written out
    // (the turns of these two loops are unrolled so that a thread's loads are issued together: a conversion right
    // behind its load holds the warp until the load has come back)
#pragma unroll 8
    for (int i = threadIdx.x; i < nb * 2 * n_state; i += blockDim.x) s_bc[i] = to_f32(bc[(size_t)t0 * 2 * n_state + i]);
#pragma unroll 4
    for (int i = threadIdx.x; i < nb * 16; i += blockDim.x) {
      const int tok = i >> 4, ch = min(c0 + (i & 15), inner - 1);
      const size_t row = (size_t)(t0 + tok);
      s_x[i] = to_f32(xc[row * inner + ch]);
      s_dt[i] = softplus_f32(dt_raw[row * inner + ch] + dt_bias[ch]);
      s_gate[i] = silu_f32(to_f32(z[row * z_ld + z_column + ch]));
    }
    __syncthreads();
#pragma unroll 4
    for (int tok = 0; tok < nb; ++tok) {      // (four tokens per turn: only S links them, the sums over lanes overlap)
      const float x = s_x[tok * 16 + grp], dt = s_dt[tok * 16 + grp];
      const float* brow = s_bc + (size_t)tok * 2 * n_state;
      const float dx = dt * x;
      float acc = 0.f;
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        const int n = sub + 8 * i;
        if (n < n_state) {
          S[i] = fmaf(expf(dt * a[i]), S[i], dx * brow[n]);
          acc = fmaf(S[i], brow[n_state + n], acc);
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (sub == 0) s_y[tok * 16 + grp] = (acc + skip * x) * s_gate[tok * 16 + grp];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < nb * 16; i += blockDim.x) {
      const int tok = i >> 4, ch = c0 + (i & 15);
      if (ch < inner) out[(size_t)(t0 + tok) * inner + ch] = from_f32<T>(s_y[i]);
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int n = sub + 8 * i;
      if (n < n_state) st[n] = S[i];
    }
  }
}

// ------------------------------------------------------------------ gated delta rule
// Per value head h (query/key head c = h / (heads / kv_heads)) and token, with k, q scaled to unit length
// (q also by q_scale), beta = sigmoid(b), g = exp(-rate[h] * softplus(a + dt_bias[h])):
//     S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q.
// A column S[:, j] is independent of the others: eight lanes share a column, lane l holding the row pairs
// (16 m + 2 l, 16 m + 2 l + 1), m = 0 .. RPL / 2 - 1, as float2 values, so that the products, decays and updates of a
// token are the two-wide float32 instructions of sm_100 (__ffma2_rn and __fmul2_rn round each half like the scalar
// forms) and k and q come from shared memory as 8-byte packets.  A block of 128 threads walks 16 columns of one head of
// one request through its tokens.
// The tokens come in batches of kDeltaBatch.  All threads bring a batch's q and k of the head (once, not once per
// column), its 16 values, gates and decays into shared memory, and hold the next batch's q and k in registers while the
// current one is walked, so that the walk, whose steps depend on one another, never waits for global memory.  The unit
// scaling is folded into the walk: with kn = 1 / |k| and qn = q_scale / |q|,
//     dot = kn * (S^T k);  u = beta (v - dot);  S <- S + k (kn u);  o = qn * (S^T q).
// qkv rows: [q: kv_heads * d | k: kv_heads * d | v: heads * dv];  ba rows: [b: heads | a: heads] float32.
// Shared memory: kDeltaBatch * (2 * 8 * RPL + 16 + 4) floats; rows of q and k are 8 * RPL floats apart, zero beyond d.
constexpr int kDeltaBatch = 16;

template <typename T, int RPL>
__global__ void __launch_bounds__(128)
gated_delta_rule_kernel(float* __restrict__ out, const T* __restrict__ qkv, const float* __restrict__ ba,
                        const float* __restrict__ rate, const float* __restrict__ dt_bias, float* __restrict__ state,
                        const int* __restrict__ q_start, const int* __restrict__ positions, const int* __restrict__ state_slot,
                        int heads, int kv_heads, int d, int dv, float unit_eps, float q_scale) {
  static_assert(RPL % 2 == 0, "a lane holds pairs of rows");
  constexpr int DS = 8 * RPL;                       // floats between rows of q and k in shared memory
  constexpr int HP = RPL / 2;                       // row pairs of a lane
  extern __shared__ __align__(16) float delta_smem[];
  float* s_q = delta_smem;                         // [batch][DS], as projected
  float* s_k = s_q + kDeltaBatch * DS;
  float* s_v = s_k + kDeltaBatch * DS;             // [batch][16]
  float* s_beta = s_v + kDeltaBatch * 16;
  float* s_g = s_beta + kDeltaBatch;
  float* s_qn = s_g + kDeltaBatch;
  float* s_kn = s_qn + kDeltaBatch;
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.z, h = blockIdx.y;
  const int lo = q_start[r], hi = q_start[r + 1];
  if (hi <= lo || state_slot[r] < 0) return;
  const int sub = threadIdx.x & 7, grp = threadIdx.x >> 3;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int j0 = blockIdx.x * 16;
  const bool live = j0 + grp < dv;
  const int j = live ? j0 + grp : dv - 1;
  const int c = h / (heads / kv_heads);
  const int ld = 2 * kv_heads * d + heads * dv;
  float* st = state + (((size_t)state_slot[r] * heads + h) * d) * dv + j;
  const bool from_zero = positions[lo] == 0;
  float2 S[HP];
#pragma unroll
  for (int m = 0; m < HP; ++m) {
    const int row = 16 * m + 2 * sub;
    S[m].x = (row < d && !from_zero) ? st[(size_t)row * dv] : 0.f;
    S[m].y = (row + 1 < d && !from_zero) ? st[(size_t)(row + 1) * dv] : 0.f;
  }
  for (int i = threadIdx.x; i < 2 * kDeltaBatch * DS; i += blockDim.x) s_q[i] = 0.f;   // (s_k follows s_q) zero beyond d for good
  const float rate_h = rate[h], bias_h = dt_bias[h];
  // Element i of a thread's share of a batch: flat index threadIdx.x + 128 * i over [batch][d]; RPL of them cover
  // kDeltaBatch * d = 16 d <= 128 * RPL (d <= 8 * RPL).  (token, element) of the flat index advance without a division.
  // They are kept as fetched (T, not float): a conversion right behind its load would hold the warp until the load has
  // come back, and the point is to have the loads in flight during the walk.  The same for the batch's 16 x 16 values
  // (two per thread) and a token's two gate inputs.
  T pq[RPL], pk[RPL], pv[2];
  float pb = 0.f, pa = 0.f;
  const int tok_first = threadIdx.x / d, e_first = threadIdx.x % d, tok_step = 128 / d, e_step = 128 % d;
  auto fetch = [&](int t0) {
    const int nb = min(kDeltaBatch, hi - t0);
    int tok = tok_first, e = e_first;
#pragma unroll
    for (int i = 0; i < RPL; ++i) {
      if (tok < nb) {
        const T* row = qkv + (size_t)(t0 + tok) * ld;
        pq[i] = row[c * d + e];
        pk[i] = row[(kv_heads + c) * d + e];
      }
      tok += tok_step;
      e += e_step;
      if (e >= d) { e -= d; ++tok; }
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int idx = threadIdx.x + 128 * i;
      if ((idx >> 4) < nb) pv[i] = qkv[(size_t)(t0 + (idx >> 4)) * ld + 2 * kv_heads * d + h * dv + min(j0 + (idx & 15), dv - 1)];
    }
    if (threadIdx.x < nb) {
      pb = ba[(size_t)(t0 + threadIdx.x) * 2 * heads + h];
      pa = ba[(size_t)(t0 + threadIdx.x) * 2 * heads + heads + h];
    }
  };
  fetch(lo);
  for (int t0 = lo; t0 < hi; t0 += kDeltaBatch) {
    const int nb = min(kDeltaBatch, hi - t0);
    __syncthreads();                                  // the batch before has been walked (and the rows are zeroed)
    {
      int tok = tok_first, e = e_first;
#pragma unroll
      for (int i = 0; i < RPL; ++i) {
        if (tok < nb) { s_q[tok * DS + e] = to_f32(pq[i]); s_k[tok * DS + e] = to_f32(pk[i]); }
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
    if (threadIdx.x < nb) {
      s_beta[threadIdx.x] = 1.0f / (1.0f + expf(-pb));
      s_g[threadIdx.x] = expf(-rate_h * softplus_f32(pa + bias_h));
    }
    __syncthreads();
    if (t0 + kDeltaBatch < hi) fetch(t0 + kDeltaBatch);   // in flight while this batch is walked
    {
      // the lengths of q and k: warp w takes tokens w, w + 4, w + 8, w + 12, their eight sums over the lanes side by side
      float qq[4] = {0.f, 0.f, 0.f, 0.f}, kk[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const int tok = warp + 4 * m;
        if (tok < nb)
          for (int e = lane; e < d; e += 32) {
            qq[m] = fmaf(s_q[tok * DS + e], s_q[tok * DS + e], qq[m]);
            kk[m] = fmaf(s_k[tok * DS + e], s_k[tok * DS + e], kk[m]);
          }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
        for (int m = 0; m < 4; ++m) {
          qq[m] += __shfl_xor_sync(0xffffffffu, qq[m], o);
          kk[m] += __shfl_xor_sync(0xffffffffu, kk[m], o);
        }
      }
#pragma unroll
      for (int m = 0; m < 4; ++m) {
        const int tok = warp + 4 * m;
        if (lane == 0 && tok < nb) {
          s_qn[tok] = q_scale / sqrtf(qq[m] + unit_eps);
          s_kn[tok] = 1.0f / sqrtf(kk[m] + unit_eps);
        }
      }
    }
    __syncthreads();
#pragma unroll (RPL <= 16 ? 2 : 1)
    for (int tok = 0; tok < nb; ++tok) {      // (two tokens per turn: the read-out of one overlaps the update of the next)
      const float2* kp = reinterpret_cast<const float2*>(s_k + tok * DS) + sub;     // pair m of this lane: kp[8 * m]
      const float2* qp = reinterpret_cast<const float2*>(s_q + tok * DS) + sub;
      const float g = s_g[tok], kn = s_kn[tok];
      const float2 g2 = make_float2(g, g);
      float2 k[HP];
      float2 dot0 = make_float2(0.f, 0.f), dot1 = make_float2(0.f, 0.f);
#pragma unroll
      for (int m = 0; m < HP; ++m) {
        k[m] = kp[8 * m];
        S[m] = __fmul2_rn(S[m], g2);
        if (m & 1) dot1 = __ffma2_rn(S[m], k[m], dot1); else dot0 = __ffma2_rn(S[m], k[m], dot0);
      }
      float dot = (dot0.x + dot0.y) + (dot1.x + dot1.y);
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float u = s_beta[tok] * (s_v[tok * 16 + grp] - kn * dot) * kn;
      const float2 u2 = make_float2(u, u);
      float2 acc0 = make_float2(0.f, 0.f), acc1 = make_float2(0.f, 0.f);
#pragma unroll
      for (int m = 0; m < HP; ++m) {
        S[m] = __ffma2_rn(k[m], u2, S[m]);
        const float2 qv = qp[8 * m];
        if (m & 1) acc1 = __ffma2_rn(S[m], qv, acc1); else acc0 = __ffma2_rn(S[m], qv, acc0);
      }
      float acc = (acc0.x + acc0.y) + (acc1.x + acc1.y);
#pragma unroll
      for (int o = 1; o < 8; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (sub == 0 && live) out[(size_t)(t0 + tok) * heads * dv + h * dv + j] = acc * s_qn[tok];
    }
  }
  if (live) {
#pragma unroll
    for (int m = 0; m < HP; ++m) {
      const int row = 16 * m + 2 * sub;
      if (row < d) st[(size_t)row * dv] = S[m].x;
      if (row + 1 < d) st[(size_t)(row + 1) * dv] = S[m].y;
    }
  }
}

// ------------------------------------------------------------------ per-head norm with an output gate
// out[t, column + h * dv + e] = o[t, h, e] * rsqrt(mean_e(o^2) + eps) * w[e] * silu(gate[t, gate_column + h * dv + e]) * scale.
// With `sigmoid_gate` the gate passes a sigmoid instead of silu; with `weight_per_head` the weight is w[h * dv + e].
// One warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(256)
gated_head_norm_kernel(T* __restrict__ out, int out_ld, int column, const float* __restrict__ o, const float* __restrict__ w,
                       float eps, const T* __restrict__ gate, int gate_ld, int gate_column, int tokens, int heads, int dv,
                       float scale, int sigmoid_gate, int weight_per_head) {
  pdl_wait();
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const size_t item = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= (size_t)tokens * heads) return;
  const int t = (int)(item / heads), h = (int)(item % heads);
  const float* src = o + (size_t)t * heads * dv + (size_t)h * dv;
  float ss = 0.f;
#pragma unroll 4
  for (int e = lane; e < dv; e += 32) ss = fmaf(src[e], src[e], ss);
  ss = warp_sum(ss);
  const float rrms = 1.0f / sqrtf(ss / (float)dv + eps);
  const float* wh = weight_per_head ? w + (size_t)h * dv : w;
#pragma unroll 4
  for (int e = lane; e < dv; e += 32) {
    const float g = to_f32(gate[(size_t)t * gate_ld + gate_column + h * dv + e]);
    const float gated = sigmoid_gate ? 1.0f / (1.0f + expf(-g)) : silu_f32(g);
    out[(size_t)t * out_ld + column + h * dv + e] = from_f32<T>(src[e] * rrms * wh[e] * gated * scale);
  }
}

// ------------------------------------------------------------------ launchers
template <typename T>
int causal_conv(void* out, const void* x, int ld, int column, int channels, const float* w, const float* b, int taps, float* state,
                const int* q_start, const int* tok_req, const int* positions, const int* state_slot, int tokens, int requests,
                int silu, int single_tokens, void* stream) {
  PTL_REQUIRE(tokens >= 0 && requests >= 0 && channels > 0 && taps > 0 && column >= 0 && column + channels <= ld,
              "causal_conv: bad sizes tokens=%d channels=%d taps=%d column=%d ld=%d", tokens, channels, taps, column, ld);
  if (tokens == 0) return 0;
  const dim3 block(128), tiles((channels + 127) / 128);
  PTL_REQUIRE(tiles.x <= 65535, "causal_conv: too many channels (%d)", channels);
  // a step of single tokens (as many rows as requests, each request's rows being one): one kernel reads and moves the state
  float* state_out = (single_tokens && taps > 1) ? state : nullptr;
  if (int rc = launch_kernel("causal_conv", causal_conv_kernel<T>, dim3(tokens, tiles.x), block, 0, as_stream(stream), (T*)out,
                             (const T*)x, ld, column, channels, w, b, taps, (const float*)state, q_start, tok_req, positions,
                             state_slot, silu, state_out))
    return rc;
  if (taps == 1 || requests == 0 || state_out) return 0;
  return launch_kernel("conv_state", conv_state_kernel<T>, dim3(requests, tiles.x), block, 0, as_stream(stream), state, (const T*)x,
                       ld, column, channels, taps, q_start, positions, state_slot);
}

template <typename T>
int selective_scan(void* out, const void* xc, const float* dt_raw, const float* dt_bias, const float* A, const void* bc,
                   const float* D, const void* z, int z_ld, int z_column, int inner, int n_state, float* state, const int* q_start,
                   const int* positions, const int* state_slot, int requests, void* stream) {
  PTL_REQUIRE(requests >= 0 && inner > 0 && n_state > 0 && n_state <= 256 && z_column >= 0 && z_column + inner <= z_ld,
              "selective_scan: bad sizes inner=%d state=%d (at most 256)", inner, n_state);
  PTL_REQUIRE(requests <= 65535, "selective_scan: at most 65535 requests per step, got %d", requests);
  if (requests == 0) return 0;
  const dim3 grid((inner + 15) / 16, requests), block(128);
  const int tb = n_state <= 64 ? 32 : (n_state <= 128 ? 16 : 8);          // at most 20 KB of shared memory
  const size_t smem = (size_t)tb * (2 * n_state + 64) * sizeof(float);
#define PTL_SCAN(NPL) return launch_kernel("selective_scan", selective_scan_kernel<T, NPL>, grid, block, smem, as_stream(stream), \
    (T*)out, (const T*)xc, dt_raw, dt_bias, A, (const T*)bc, D, (const T*)z, z_ld, z_column, inner, n_state, state, q_start, \
    positions, state_slot, tb)
  const int per_lane = (n_state + 7) / 8;
  if (per_lane <= 1) PTL_SCAN(1);
  if (per_lane <= 2) PTL_SCAN(2);
  if (per_lane <= 3) PTL_SCAN(3);
  if (per_lane <= 4) PTL_SCAN(4);
  if (per_lane <= 8) PTL_SCAN(8);
  if (per_lane <= 16) PTL_SCAN(16);
  PTL_SCAN(32);
#undef PTL_SCAN
}

template <typename T>
int gated_delta_rule(float* out, const void* qkv, const float* ba, const float* rate, const float* dt_bias, float* state,
                     const int* q_start, const int* positions, const int* state_slot, int requests, int heads, int kv_heads, int d,
                     int dv, float unit_eps, float q_scale, void* stream) {
  PTL_REQUIRE(requests >= 0 && heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && d > 0 && d <= 256 && dv > 0,
              "gated_delta_rule: bad sizes heads=%d kv_heads=%d d=%d (at most 256) dv=%d", heads, kv_heads, d, dv);
  PTL_REQUIRE(requests <= 65535 && heads <= 65535, "gated_delta_rule: at most 65535 requests and heads");
  if (requests == 0) return 0;
  const dim3 grid((dv + 15) / 16, heads, requests), block(128);
#define PTL_DELTA(RPL) return launch_kernel("gated_delta_rule", gated_delta_rule_kernel<T, RPL>, grid, block, \
    (size_t)kDeltaBatch * (2 * 8 * RPL + 16 + 4) * sizeof(float) /* at most 34 KB */, as_stream(stream), \
    out, (const T*)qkv, ba, rate, dt_bias, state, q_start, positions, state_slot, heads, kv_heads, d, dv, unit_eps, q_scale)
  const int per_lane = (d + 7) / 8;
  if (per_lane <= 2) PTL_DELTA(2);
  if (per_lane <= 4) PTL_DELTA(4);
  if (per_lane <= 8) PTL_DELTA(8);
  if (per_lane <= 12) PTL_DELTA(12);
  if (per_lane <= 16) PTL_DELTA(16);
  PTL_DELTA(32);
#undef PTL_DELTA
}

template <typename T>
int gated_head_norm(void* out, int out_ld, int column, const float* o, const float* w, float eps, const void* gate, int gate_ld,
                    int gate_column, int tokens, int heads, int dv, float scale, int sigmoid_gate, int weight_per_head, void* stream) {
  PTL_REQUIRE(tokens >= 0 && heads > 0 && dv > 0 && eps > 0.f && column >= 0 && column + heads * dv <= out_ld &&
              gate_column >= 0 && gate_column + heads * dv <= gate_ld, "gated_head_norm: bad sizes tokens=%d heads=%d dv=%d",
              tokens, heads, dv);
  if (tokens == 0) return 0;
  const size_t items = (size_t)tokens * heads;
  return launch_kernel("gated_head_norm", gated_head_norm_kernel<T>, dim3((unsigned)((items + 7) / 8)), dim3(256), 0,
                       as_stream(stream), (T*)out, out_ld, column, o, w, eps, (const T*)gate, gate_ld, gate_column, tokens, heads,
                       dv, scale, sigmoid_gate, weight_per_head);
}

}  // namespace ptl

#define PTL_RECURRENT(SUFFIX, TYPE)                                                                                               \
  PTL_EXPORT int ptl_causal_conv##SUFFIX(void* out, const void* x, int ld, int column, int channels, const float* w,               \
                                         const float* b, int taps, float* state, const int* q_start, const int* tok_req,           \
                                         const int* positions, const int* state_slot, int tokens, int requests, int silu,         \
                                         int single_tokens, void* stream) {                                                       \
    return ptl::causal_conv<TYPE>(out, x, ld, column, channels, w, b, taps, state, q_start, tok_req, positions, state_slot, tokens, \
                                  requests, silu, single_tokens, stream);                                                         \
  }                                                                                                                               \
  PTL_EXPORT int ptl_selective_scan##SUFFIX(void* out, const void* xc, const float* dt_raw, const float* dt_bias, const float* A,  \
                                            const void* bc, const float* D, const void* z, int z_ld, int z_column, int inner,      \
                                            int n_state, float* state, const int* q_start, const int* positions,                  \
                                            const int* state_slot, int requests, void* stream) {                                  \
    return ptl::selective_scan<TYPE>(out, xc, dt_raw, dt_bias, A, bc, D, z, z_ld, z_column, inner, n_state, state, q_start,        \
                                     positions, state_slot, requests, stream);                                                    \
  }                                                                                                                               \
  PTL_EXPORT int ptl_gated_delta_rule##SUFFIX(float* out, const void* qkv, const float* ba, const float* rate,                     \
                                              const float* dt_bias, float* state, const int* q_start, const int* positions,       \
                                              const int* state_slot, int requests, int heads, int kv_heads, int d, int dv,        \
                                              float unit_eps, float q_scale, void* stream) {                                      \
    return ptl::gated_delta_rule<TYPE>(out, qkv, ba, rate, dt_bias, state, q_start, positions, state_slot, requests, heads,        \
                                       kv_heads, d, dv, unit_eps, q_scale, stream);                                               \
  }                                                                                                                               \
  PTL_EXPORT int ptl_gated_head_norm##SUFFIX(void* out, int out_ld, int column, const float* o, const float* w, float eps,         \
                                             const void* gate, int gate_ld, int gate_column, int tokens, int heads, int dv,        \
                                             float scale, int sigmoid_gate, int weight_per_head, void* stream) {                  \
    return ptl::gated_head_norm<TYPE>(out, out_ld, column, o, w, eps, gate, gate_ld, gate_column, tokens, heads, dv, scale,        \
                                      sigmoid_gate, weight_per_head, stream);                                                     \
  }
PTL_RECURRENT(_f32, float)
PTL_RECURRENT(_bf16, __nv_bfloat16)
