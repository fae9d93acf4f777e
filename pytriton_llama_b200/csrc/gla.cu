// Gated linear attention: per head a float32 state S [d, dv] that decays per key channel,
//   S <- diag(a_t) S + k_t v_t^T,   o_t = S^T q_t,   a_t = sigmoid(z_t + b)^(1/tau) = exp(logsigmoid(z_t + b) / tau).
//
// With `head_decay` (and no z) every key channel of head h decays by the fixed head_decay[h] instead (retention);
// `k_scale` multiplies the keys.
//
// proj is the projection's output [T, q | k | v | ...] (H heads of d, d, dv), z float32 [T, H*d] before
// the bias.  A block owns 32 columns of one head's state for one request and walks the request's
// tokens of this step in order.  The 32 lanes of a warp are the 32 columns; each of the 8 warps holds
// every eighth packet of four of the d rows in registers, so the q, k and decay values a warp needs
// are the same for all its lanes: one shared-memory wavefront per packet.  (With 8 lanes per column
// and the rows spread over the lanes the kernel was bound by shared-memory bandwidth, 437 wavefronts a
// token.)  Nothing in the walk waits on a shuffle; the warps' partial read-outs of a batch meet in
// shared memory.  Tokens come through shared memory in batches (q scaled, decay worked out while
// staging; the next batch's values are requested before the walk over this one).  The state of a
// request is read from its slot unless the portion starts at position 0 and written back at the end.
// Everything after the loads is float32; a token's result does not depend on how the request was cut
// into steps or on what else the step holds.
#include "common.cuh"

namespace ptl {

constexpr int kGlaCols = 32;      // columns of the state per block
constexpr int kGlaLanes = 8;      // threads per column (one in each warp)
constexpr int kGlaThreads = kGlaCols * kGlaLanes;

__device__ __forceinline__ float log_sigmoid_f32(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <typename T, int RPL, int TB>   // RPL rows per lane (d <= 8 * RPL), TB tokens per batch
__global__ void __launch_bounds__(kGlaThreads)
gla_scan_kernel(float* __restrict__ out, const T* __restrict__ proj, int ld, const float* __restrict__ z,
                const float* __restrict__ bias, float inv_tau, float* __restrict__ state, const int* __restrict__ q_start,
                const int* __restrict__ positions, const int* __restrict__ state_slot, int H, int d, int dv, float q_scale,
                const float* __restrict__ head_decay, float k_scale) {
  constexpr int DP = kGlaLanes * RPL;
  __shared__ __align__(16) float s_q[TB][DP], s_k[TB][DP], s_a[TB][DP];
  __shared__ float s_v[TB][kGlaCols];
  __shared__ float s_part[TB][kGlaLanes][kGlaCols];        // a warp's part of a token's read-out, per column
  pdl_wait();
  pdl_launch_dependents();
  const int r = blockIdx.z, h = blockIdx.y;
  const int t0 = q_start[r], t1 = q_start[r + 1];
  const int slot = state_slot[r];
  if (t1 <= t0 || slot < 0) return;
  const int tid = threadIdx.x;
  const int col = tid & 31, lane8 = tid >> 5;              // column = lane; lane8: which eighth of the rows = the warp
  const int e = blockIdx.x * kGlaCols + col;
  const bool live = e < dv;
  // rows of this warp: packets of four, packet m of the warp being packet m * 8 + lane8 of the column
  auto row_of = [&](int i) { return ((i >> 2) * kGlaLanes + lane8) * 4 + (i & 3); };
  float* st = state + (((size_t)slot * H + h) * d) * dv;
  float S[RPL];
  const bool fresh = positions[t0] == 0;
#pragma unroll
  for (int i = 0; i < RPL; ++i) S[i] = (!fresh && live && row_of(i) < d) ? st[(size_t)row_of(i) * dv + e] : 0.f;
  const int qcol = h * d, kcol = H * d + h * d, vcol = 2 * H * d + h * dv + blockIdx.x * kGlaCols;
  const int vcols = min(kGlaCols, dv - blockIdx.x * kGlaCols);

  // A thread fetches the same column c of q, k and z for tokens j0, j0 + step, ...: the next batch's values are
  // requested before the walk over this batch and kept as fetched; they are converted (and the decay worked out)
  // when they go to shared memory, after the walk.
  constexpr int NE = TB * DP / kGlaThreads, NV = (TB * kGlaCols + kGlaThreads - 1) / kGlaThreads;
  constexpr int kTokStep = kGlaThreads / DP > 0 ? kGlaThreads / DP : 1;
  static_assert(kGlaThreads % DP == 0 && NE * kTokStep == TB, "a thread's column must not change between its turns");
  const int c_mine = tid % DP, j_mine = tid / DP;
  const float b_mine = (z && c_mine < d) ? bias[qcol + c_mine] : 0.f;
  const float fixed = head_decay ? head_decay[h] : 0.f;
  T rq[NE], rk[NE], rv[NV];
  float rz[NE];
  auto fetch = [&](int tb) {
    const int nt = min(TB, t1 - tb);
#pragma unroll
    for (int i = 0; i < NE; ++i) {
      const int j = j_mine + i * kTokStep;
      const bool ok = j < nt && c_mine < d;
      const T* row = proj + (size_t)(tb + (ok ? j : 0)) * ld;
      rq[i] = ok ? row[qcol + c_mine] : from_f32<T>(0.f);
      rk[i] = ok ? row[kcol + c_mine] : from_f32<T>(0.f);
      rz[i] = (ok && z) ? z[(size_t)(tb + j) * H * d + qcol + c_mine] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int idx = tid + i * kGlaThreads;
      const int j = idx / kGlaCols, c = idx % kGlaCols;
      rv[i] = (j < nt && c < vcols) ? proj[(size_t)(tb + j) * ld + vcol + c] : from_f32<T>(0.f);
    }
  };
  auto stage = [&]() {
#pragma unroll
    for (int i = 0; i < NE; ++i) {
      const int j = j_mine + i * kTokStep;
      s_q[j][c_mine] = to_f32(rq[i]) * q_scale;
      s_k[j][c_mine] = to_f32(rk[i]) * k_scale;
      s_a[j][c_mine] = c_mine < d ? (z ? expf(log_sigmoid_f32(rz[i] + b_mine) * inv_tau) : fixed) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int idx = tid + i * kGlaThreads;
      if (idx < TB * kGlaCols) s_v[idx / kGlaCols][idx % kGlaCols] = to_f32(rv[i]);
    }
  };
  fetch(t0);
  for (int tb = t0; tb < t1; tb += TB) {
    const int nt = min(TB, t1 - tb);
    __syncthreads();                       // the walk over the batch before is done with the staged tokens
    stage();
    __syncthreads();
    if (tb + TB < t1) fetch(tb + TB);
    auto token = [&](int j) {
      const float v = s_v[j][col];
      float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < RPL; i += 4) {
        const float4 a4 = *reinterpret_cast<const float4*>(&s_a[j][row_of(i)]);
        const float4 k4 = *reinterpret_cast<const float4*>(&s_k[j][row_of(i)]);
        const float4 q4 = *reinterpret_cast<const float4*>(&s_q[j][row_of(i)]);
        S[i] = fmaf(a4.x, S[i], k4.x * v);
        S[i + 1] = fmaf(a4.y, S[i + 1], k4.y * v);
        S[i + 2] = fmaf(a4.z, S[i + 2], k4.z * v);
        S[i + 3] = fmaf(a4.w, S[i + 3], k4.w * v);
        acc[0] = fmaf(q4.x, S[i], acc[0]);
        acc[1] = fmaf(q4.y, S[i + 1], acc[1]);
        acc[2] = fmaf(q4.z, S[i + 2], acc[2]);
        acc[3] = fmaf(q4.w, S[i + 3], acc[3]);
      }
      s_part[j][lane8][col] = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    };
    if (nt == TB) {
#pragma unroll 4
      for (int j = 0; j < TB; ++j) token(j);            // (unrolled: the next token's loads and products start under this one's sums)
    } else {
      for (int j = 0; j < nt; ++j) token(j);
    }
    __syncthreads();
    // the warps' parts of every read-out of the batch, added in the order of the warps
    for (int idx = tid; idx < nt * kGlaCols; idx += kGlaThreads) {
      const int j = idx / kGlaCols, c = idx % kGlaCols;
      float sum = 0.f;
#pragma unroll
      for (int w = 0; w < kGlaLanes; ++w) sum += s_part[j][w][c];
      if (c < vcols) out[(size_t)(tb + j) * H * dv + (size_t)h * dv + blockIdx.x * kGlaCols + c] = sum;
    }
  }
  if (live) {
#pragma unroll
    for (int i = 0; i < RPL; ++i)
      if (row_of(i) < d) st[(size_t)row_of(i) * dv + e] = S[i];
  }
}

template <typename T>
int gla_scan(float* out, const void* proj, int ld, const float* z, const float* bias, float inv_tau, float* state,
             const int* q_start, const int* positions, const int* state_slot, int requests, int H, int d, int dv,
             float q_scale, const float* head_decay, float k_scale, void* stream) {
  PTL_REQUIRE(requests >= 0 && H > 0 && d > 0 && dv > 0, "gla_scan: bad sizes");
  PTL_REQUIRE((z && bias) || head_decay, "gla_scan: neither a decay per channel nor one per head");
  PTL_REQUIRE(d <= 256, "gla_scan: head size %d, at most 256", d);
  PTL_REQUIRE(ld >= 2 * H * d + H * dv, "gla_scan: rows of %d elements are too short", ld);
  PTL_REQUIRE(H <= 65535 && requests <= 65535, "gla_scan: too many heads or requests");
  if (requests == 0) return 0;
  const dim3 grid((dv + kGlaCols - 1) / kGlaCols, H, requests), block(kGlaThreads);
#define PTL_GLA_LAUNCH(RPL, TB)                                                                                              \
  return launch_kernel("gla_scan", gla_scan_kernel<T, RPL, TB>, grid, block, 0, as_stream(stream), out, (const T*)proj, ld, z, \
                       bias, inv_tau, state, q_start, positions, state_slot, H, d, dv, q_scale, z ? nullptr : head_decay, k_scale)
  if (d <= 32) PTL_GLA_LAUNCH(4, 16);
  if (d <= 64) PTL_GLA_LAUNCH(8, 16);
  if (d <= 128) PTL_GLA_LAUNCH(16, 16);
  PTL_GLA_LAUNCH(32, 8);
#undef PTL_GLA_LAUNCH
}

}  // namespace ptl

#define PTL_GLA(SUFFIX, TYPE)                                                                                                   \
  PTL_EXPORT int ptl_gla_scan##SUFFIX(float* out, const void* proj, int ld, const float* z, const float* bias, float inv_tau,    \
                                      float* state, const int* q_start, const int* positions, const int* state_slot,            \
                                      int requests, int H, int d, int dv, float q_scale, const float* head_decay,               \
                                      float k_scale, void* stream) {                                                            \
    return ptl::gla_scan<TYPE>(out, proj, ld, z, bias, inv_tau, state, q_start, positions, state_slot, requests, H, d, dv,       \
                               q_scale, head_decay, k_scale, stream);                                                           \
  }
PTL_GLA(_f32, float)
PTL_GLA(_bf16, __nv_bfloat16)
