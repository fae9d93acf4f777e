// out[M, N] (+)= A[M, K] * W[N, K]^T on the CUDA cores in float32: the true 32-bit matrix product
// of the float32 path (no tensor-core mode that drops mantissa bits), and a library-free check for
// the bfloat16 tensor-core kernels.  Any M, N, K; both operands are K-contiguous.
// A launch may hold several products of one shape (blockIdx.z = b): operand and result pointers move on by
// batch_a, batch_w, batch_o elements per b (the heads of an activation [M, heads * x] against weights
// [heads, N, K]); with `gate` the result of row m of product b is multiplied by sigmoid(gate[m * gate_ld + b]).
//
// Summation order, the same for every tile shape, so that a row's result does not depend on how
// many rows the call has (a prompt portion and a single decoded token give the same bits):
// the K range is cut into chunks of 32; inside a chunk the products are added one by one with
// fused multiply-adds, k ascending, into a fresh accumulator; the chunk sums are added to the
// running total with a compensated (Kahan) addition.  A plain running sum over K = 8,192 terms is
// wrong by about K/4 ulp of a term, which over 16 layers of a 2,048-wide model reaches 3e-4 in the
// logits; with chunks the error of a product is that of one chunk, a few ulp.
#include "common.cuh"

namespace ptl {

constexpr int kSimtChunk = 32;       // k values per chunk: the tile depth of every kernel shape

// sum += chunk, with the rounding error of the addition carried in `comp`
__device__ __forceinline__ void kahan_add(float& sum, float& comp, float chunk) {
  const float y = __fsub_rn(chunk, comp);
  const float t = __fadd_rn(sum, y);
  comp = __fsub_rn(__fsub_rn(t, sum), y);
  sum = t;
}

template <typename TI, typename TO, int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__((BM / TM) * (BN / TN))
gemm_simt_kernel(TO* __restrict__ out, const TI* __restrict__ A, const TI* __restrict__ W,
                 int M, int N, int K, int lda, int ldw, int ldo, int accumulate, int vec_ok,
                 long long batch_a, long long batch_w, long long batch_o, const TI* __restrict__ gate, int gate_ld) {
  constexpr int BK = kSimtChunk;
  constexpr int THREADS = (BM / TM) * (BN / TN);
  static_assert(TM % 4 == 0 || TM == 2 || TM == 1, "rows per thread");
  pdl_wait();
  pdl_launch_dependents();
  A += (size_t)blockIdx.z * batch_a;
  W += (size_t)blockIdx.z * batch_w;
  out += (size_t)blockIdx.z * batch_o;
  __shared__ __align__(16) float As[BK][BM + 4];
  __shared__ __align__(16) float Ws[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid % (BN / TN);  // along N
  const int ty = tid / (BN / TN);  // along M
  const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
  float acc[TM][TN], sum[TM][TN], comp[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) { sum[i][j] = 0.f; comp[i][j] = 0.f; }

  for (int k0 = 0; k0 < K; k0 += BK) {
    if (vec_ok) {
      // float32 operands whose rows start on 16-byte boundaries: four k values per load
      if constexpr (sizeof(TI) == 4) {
        for (int e = tid; e < BM * (BK / 4); e += THREADS) {
          const int r = e / (BK / 4), c4 = e % (BK / 4);
          const int gm = m0 + r, gk = k0 + c4 * 4;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (gm < M && gk < K) v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(A) + (size_t)gm * lda + gk);
          As[c4 * 4 + 0][r] = v.x; As[c4 * 4 + 1][r] = v.y; As[c4 * 4 + 2][r] = v.z; As[c4 * 4 + 3][r] = v.w;
        }
        for (int e = tid; e < BN * (BK / 4); e += THREADS) {
          const int r = e / (BK / 4), c4 = e % (BK / 4);
          const int gn = n0 + r, gk = k0 + c4 * 4;
          float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
          if (gn < N && gk < K) v = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(W) + (size_t)gn * ldw + gk);
          Ws[c4 * 4 + 0][r] = v.x; Ws[c4 * 4 + 1][r] = v.y; Ws[c4 * 4 + 2][r] = v.z; Ws[c4 * 4 + 3][r] = v.w;
        }
      }
    } else {
      // any element type and alignment: consecutive threads walk along K so that global reads coalesce
      for (int e = tid; e < BM * BK; e += THREADS) {
        const int r = e / BK, c = e % BK;
        const int gm = m0 + r, gk = k0 + c;
        As[c][r] = (gm < M && gk < K) ? to_f32(A[(size_t)gm * lda + gk]) : 0.f;
      }
      for (int e = tid; e < BN * BK; e += THREADS) {
        const int r = e / BK, c = e % BK;
        const int gn = n0 + r, gk = k0 + c;
        Ws[c][r] = (gn < N && gk < K) ? to_f32(W[(size_t)gn * ldw + gk]) : 0.f;
      }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[kk][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) kahan_add(sum[i][j], comp[i][j], acc[i][j]);
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int gm = m0 + ty * TM + i;
    if (gm >= M) continue;
    const float row_gate = gate ? 1.0f / (1.0f + expf(-to_f32(gate[(size_t)gm * gate_ld + blockIdx.z]))) : 1.0f;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int gn = n0 + tx * TN + j;
      if (gn >= N) continue;
      TO* o = out + (size_t)gm * ldo + gn;
      float v = sum[i][j] * row_gate;
      if (accumulate) v += to_f32(*o);
      *o = from_f32<TO>(v);
    }
  }
}

template <typename TI, typename TO>
int gemm_simt(void* out, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldo,
              int accumulate, void* stream, int batch = 1, long long batch_a = 0, long long batch_w = 0, long long batch_o = 0,
              const void* gate_v = nullptr, int gate_ld = 0) {
  PTL_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_simt: bad sizes M=%d N=%d K=%d", M, N, K);
  PTL_REQUIRE(lda >= K && ldw >= K && ldo >= N, "gemm_simt: pitches smaller than rows");
  PTL_REQUIRE(batch >= 1 && batch <= 65535, "gemm_simt: %d products in one launch", batch);
  if (M == 0) return 0;
  const TI* gate = (const TI*)gate_v;
  const int vec_ok = sizeof(TI) == 4 && K % 4 == 0 && lda % 4 == 0 && ldw % 4 == 0 && aligned16(A) && aligned16(W) &&
                     batch_a % 4 == 0 && batch_w % 4 == 0;
  if (M > 32) {
    constexpr int BM = 128, BN = 64, TM = 8, TN = 4;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, batch);
    PTL_REQUIRE(grid.y <= 65535, "gemm_simt: M=%d too large", M);
    return launch_kernel("gemm_simt", gemm_simt_kernel<TI, TO, BM, BN, TM, TN>, grid, dim3((BM / TM) * (BN / TN)), 0,
                         as_stream(stream), (TO*)out, (const TI*)A, (const TI*)W, M, N, K, lda, ldw, ldo, accumulate, vec_ok,
                         batch_a, batch_w, batch_o, gate, gate_ld);
  } else {
    // few rows: narrow tiles so that the weight matrix is spread over many blocks
    constexpr int BM = 32, BN = 16, TM = 4, TN = 1;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, batch);
    return launch_kernel("gemm_simt", gemm_simt_kernel<TI, TO, BM, BN, TM, TN>, grid, dim3((BM / TM) * (BN / TN)), 0,
                         as_stream(stream), (TO*)out, (const TI*)A, (const TI*)W, M, N, K, lda, ldw, ldo, accumulate, vec_ok,
                         batch_a, batch_w, batch_o, gate, gate_ld);
  }
}

// The heads' products of a step with few tokens, 16-bit operands: a warp per output feature o of a head reads the weight
// row W[b, o, :] once, in packets of 16 bytes, against up to kHfTok token rows held as float32 in shared memory;
// float32 sums, each (token, feature) by the same chain whatever else the step holds: a lane adds its packets in order,
// the lanes meet in a butterfly.  K a multiple of 8, every row on a 16-byte boundary.
constexpr int kHfTok = 8, kHfWarps = 8;

template <typename T>
__global__ void __launch_bounds__(kHfWarps * 32)
head_linear_few_kernel(T* __restrict__ out, const T* __restrict__ A, const T* __restrict__ W, int M, int N, int K, int lda, int ldo,
                       int batch_a, int batch_o, const T* __restrict__ gate, int gate_ld) {
  extern __shared__ __align__(16) float hf_x[];          // [kHfTok][K]
  pdl_wait();
  pdl_launch_dependents();
  const int b = blockIdx.y, m0 = blockIdx.z * kHfTok;
  const int nt = min(kHfTok, M - m0);
  const int packets = K / 8;
  for (int idx = threadIdx.x; idx < kHfTok * packets; idx += blockDim.x) {
    const int t = idx / packets, pk = idx % packets;
    float4 lo = make_float4(0.f, 0.f, 0.f, 0.f), hi = lo;
    if (t < nt) {
      const uint4 raw = *reinterpret_cast<const uint4*>(A + (size_t)(m0 + t) * lda + (size_t)b * batch_a + 8 * pk);
      const T* v = reinterpret_cast<const T*>(&raw);
      lo = make_float4(to_f32(v[0]), to_f32(v[1]), to_f32(v[2]), to_f32(v[3]));
      hi = make_float4(to_f32(v[4]), to_f32(v[5]), to_f32(v[6]), to_f32(v[7]));
    }
    float4* dst = reinterpret_cast<float4*>(hf_x + (size_t)t * K + 8 * pk);
    dst[0] = lo;
    dst[1] = hi;
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int o = blockIdx.x * kHfWarps + warp;
  if (o >= N) return;
  const T* wr = W + ((size_t)b * N + o) * K;
  float acc[kHfTok];
#pragma unroll
  for (int t = 0; t < kHfTok; ++t) acc[t] = 0.f;
  for (int i = lane * 8; i < K; i += 256) {
    const uint4 raw = *reinterpret_cast<const uint4*>(wr + i);
    const T* v = reinterpret_cast<const T*>(&raw);
    float w[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) w[e] = to_f32(v[e]);
#pragma unroll
    for (int t = 0; t < kHfTok; ++t) {
      const float4* xp = reinterpret_cast<const float4*>(hf_x + (size_t)t * K + i);
      const float4 x0 = xp[0], x1 = xp[1];
      float a = acc[t];
      a = fmaf(w[0], x0.x, a); a = fmaf(w[1], x0.y, a); a = fmaf(w[2], x0.z, a); a = fmaf(w[3], x0.w, a);
      a = fmaf(w[4], x1.x, a); a = fmaf(w[5], x1.y, a); a = fmaf(w[6], x1.z, a); a = fmaf(w[7], x1.w, a);
      acc[t] = a;
    }
  }
#pragma unroll
  for (int t = 0; t < kHfTok; ++t) {
    const float v = warp_sum(acc[t]);
    if (lane == t && t < nt) {
      const size_t m = (size_t)(m0 + t);
      const float g = gate ? 1.0f / (1.0f + expf(-to_f32(gate[m * gate_ld + b]))) : 1.0f;
      out[m * ldo + (size_t)b * batch_o + o] = from_f32<T>(v * g);
    }
  }
}

template <typename T>
int head_linear_few(void* out, const void* A, const void* W, int M, int N, int K, int lda, int ldo, int heads, int batch_a,
                    int batch_o, const void* gate, int gate_ld, void* stream) {
  PTL_REQUIRE(M >= 0 && N > 0 && K > 0 && heads >= 1 && heads <= 65535, "head_linear_few: bad sizes M=%d N=%d K=%d", M, N, K);
  PTL_REQUIRE(sizeof(T) == 2 && K % 8 == 0 && lda % 8 == 0 && batch_a % 8 == 0 && aligned16(A) && aligned16(W) &&
                  (size_t)kHfTok * K * sizeof(float) <= 48 * 1024,
              "head_linear_few: 16-bit rows of whole packets of 16 bytes on 16-byte boundaries, K=%d at most 1536", K);
  if (M == 0) return 0;
  const dim3 grid((N + kHfWarps - 1) / kHfWarps, heads, (M + kHfTok - 1) / kHfTok);
  PTL_REQUIRE(grid.z <= 65535, "head_linear_few: M=%d too large", M);
  return launch_kernel("head_linear_few", head_linear_few_kernel<T>, grid, dim3(kHfWarps * 32), (size_t)kHfTok * K * sizeof(float),
                       as_stream(stream), (T*)out, (const T*)A, (const T*)W, M, N, K, lda, ldo, batch_a, batch_o, (const T*)gate,
                       gate_ld);
}

}  // namespace ptl

PTL_EXPORT int ptl_gemm_simt_f32(void* out, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldo, int accumulate, void* stream) {
  return ptl::gemm_simt<float, float>(out, A, W, M, N, K, lda, ldw, ldo, accumulate, stream);
}
PTL_EXPORT int ptl_gemm_simt_bf16(void* out, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldo, int accumulate, void* stream) {
  return ptl::gemm_simt<__nv_bfloat16, __nv_bfloat16>(out, A, W, M, N, K, lda, ldw, ldo, accumulate, stream);
}
PTL_EXPORT int ptl_gemm_simt_bf16_f32out(void* out, const void* A, const void* W, int M, int N, int K, int lda, int ldw, int ldo, int accumulate, void* stream) {
  return ptl::gemm_simt<__nv_bfloat16, float>(out, A, W, M, N, K, lda, ldw, ldo, accumulate, stream);
}

// The heads of an activation against per-head weights: for b < heads,
//   out[m, b * batch_o + n] = sum_k A[m, b * batch_a + k] * W[b, n, k]   (times sigmoid(gate[m * gate_ld + b]) with a gate).
PTL_EXPORT int ptl_head_linear_f32(void* out, const void* A, const void* W, int M, int N, int K, int lda, int ldo, int heads,
                                   int batch_a, int batch_o, const void* gate, int gate_ld, void* stream) {
  return ptl::gemm_simt<float, float>(out, A, W, M, N, K, lda, K, ldo, 0, stream, heads, batch_a, (long long)N * K, batch_o, gate, gate_ld);
}
PTL_EXPORT int ptl_head_linear_bf16(void* out, const void* A, const void* W, int M, int N, int K, int lda, int ldo, int heads,
                                    int batch_a, int batch_o, const void* gate, int gate_ld, void* stream) {
  return ptl::gemm_simt<__nv_bfloat16, __nv_bfloat16>(out, A, W, M, N, K, lda, K, ldo, 0, stream, heads, batch_a, (long long)N * K,
                                                      batch_o, gate, gate_ld);
}
PTL_EXPORT int ptl_head_linear_few_bf16(void* out, const void* A, const void* W, int M, int N, int K, int lda, int ldo, int heads,
                                        int batch_a, int batch_o, const void* gate, int gate_ld, void* stream) {
  return ptl::head_linear_few<__nv_bfloat16>(out, A, W, M, N, K, lda, ldo, heads, batch_a, batch_o, gate, gate_ld, stream);
}
