// Layer norm with weight and bias, fused with the residual add, and the xIELU activation.
//
// add_layernorm, per output row m (r = rows ? rows[m] : m):
//   s = residual_in[r] + x[r] + add_bias        (each term optional; s is float32)
//   residual_out[m] = s                         (when given)
//   y[m] = (s - mean(s)) * rsqrt(mean((s - mean(s))^2) + eps) * w + b
// The mean is taken first and the squared deviations are summed in a second walk over the row, which
// is held in shared memory: float32 throughout, no difference of two large sums.  One block per row.
// TX is the element type of x, TY that of y (float32 y from bfloat16 x: the norm an embedding passes
// on its way to becoming the float32 stream).
//
// xielu, elementwise in float32:  z > 0: ap z^2 + z / 2;   z <= 0: aq (expm1(z) - z) + z / 2.
#include "common.cuh"

namespace ptl {

template <typename TX, typename TY>
__global__ void __launch_bounds__(256)
add_layernorm_kernel(TY* __restrict__ y, float* __restrict__ residual_out, const float* __restrict__ residual_in,
                     const TX* __restrict__ x, const float* __restrict__ add_bias, const float* __restrict__ w,
                     const float* __restrict__ b, const int* __restrict__ rows, int hidden, float eps) {
  extern __shared__ float ln_row[];
  __shared__ float red[33];
  pdl_wait();
  pdl_launch_dependents();
  const int m = blockIdx.x;
  const int r = rows ? rows[m] : m;
  const float* rin = residual_in ? residual_in + (size_t)r * hidden : nullptr;
  const TX* xin = x ? x + (size_t)r * hidden : nullptr;
  float* rout = residual_out ? residual_out + (size_t)m * hidden : nullptr;
  TY* yo = y + (size_t)m * hidden;
  float sum = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float s = rin ? rin[i] : 0.f;
    if (xin) s += to_f32(xin[i]);
    if (add_bias) s += add_bias[i];
    ln_row[i] = s;
    if (rout && (xin || add_bias || rout != rin)) rout[i] = s;      // unchanged rows are not rewritten
    sum += s;
  }
  const float mean = block_sum(sum, red) / (float)hidden;
  float sq = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    const float dlt = ln_row[i] - mean;
    sq = fmaf(dlt, dlt, sq);
  }
  const float rstd = 1.0f / sqrtf(block_sum(sq, red) / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    yo[i] = from_f32<TY>(fmaf((ln_row[i] - mean) * rstd, w[i], b[i]));
}

template <typename TX, typename TY>
int add_layernorm(void* y, float* residual_out, const float* residual_in, const void* x, const float* add_bias, const float* w,
                  const float* b, const int* rows, int out_rows, int hidden, float eps, void* stream) {
  PTL_REQUIRE(out_rows >= 0 && hidden > 0 && eps > 0.f && w && b && (x || residual_in), "add_layernorm: bad arguments");
  PTL_REQUIRE((size_t)hidden * sizeof(float) <= 200 * 1024, "add_layernorm: rows of %d do not fit shared memory", hidden);
  if (out_rows == 0) return 0;
  const size_t smem = (size_t)hidden * sizeof(float);
  static SmemRaised raised;
  if (smem > 48 * 1024)
    if (int rc = raise_shared_memory("add_layernorm", add_layernorm_kernel<TX, TY>, 200 * 1024, raised)) return rc;
  return launch_kernel("add_layernorm", add_layernorm_kernel<TX, TY>, dim3(out_rows), dim3(256), smem, as_stream(stream), (TY*)y,
                       residual_out, residual_in, (const TX*)x, add_bias, w, b, rows, hidden, eps);
}

// FAST (16-bit results): e^z - 1 by the fast exponential; its absolute error, 2^-22 or so, is far below the rounding of the
// result, which z / 2 dominates where e^z - 1 - z is small.
template <bool FAST>
__device__ __forceinline__ float xielu_f32(float z, float ap, float aq) {
  const float em1 = FAST ? __expf(z) - 1.0f : expm1f(z);
  return z > 0.f ? fmaf(ap * z, z, 0.5f * z) : fmaf(aq, em1 - z, 0.5f * z);
}

// A thread takes one packet of 16 bytes (PER elements); the elements after the last whole packet go one by one.
template <typename T>
__global__ void __launch_bounds__(256) xielu_kernel(T* __restrict__ out, const T* __restrict__ x, long long n, long long packets,
                                                    float ap, float aq) {
  constexpr int PER = 16 / sizeof(T);
  pdl_wait();
  pdl_launch_dependents();
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < packets) {
    uint4 raw = reinterpret_cast<const uint4*>(x)[i];
    T* v = reinterpret_cast<T*>(&raw);
#pragma unroll
    for (int e = 0; e < PER; ++e) v[e] = from_f32<T>(xielu_f32<sizeof(T) == 2>(to_f32(v[e]), ap, aq));
    reinterpret_cast<uint4*>(out)[i] = raw;
  } else {
    const long long j = packets * PER + (i - packets);
    if (j < n) out[j] = from_f32<T>(xielu_f32<sizeof(T) == 2>(to_f32(x[j]), ap, aq));
  }
}

template <typename T>
int xielu(void* out, const void* x, long long n, float ap, float aq, void* stream) {
  PTL_REQUIRE(n >= 0, "xielu: bad size");
  if (n == 0) return 0;
  constexpr int PER = 16 / sizeof(T);
  const long long packets = (aligned16(out) && aligned16(x)) ? n / PER : 0;
  const long long threads = packets + (n - packets * PER);
  return launch_kernel("xielu", xielu_kernel<T>, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, as_stream(stream), (T*)out,
                       (const T*)x, n, packets, ap, aq);
}

}  // namespace ptl

// y_f32: y is float32 whatever the element type of x
#define PTL_LAYERNORM(SUFFIX, TYPE)                                                                                               \
  PTL_EXPORT int ptl_add_layernorm##SUFFIX(void* y, float* residual_out, const float* residual_in, const void* x,                  \
                                           const float* add_bias, const float* w, const float* b, const int* rows, int out_rows,  \
                                           int hidden, float eps, int y_f32, void* stream) {                                      \
    if (y_f32)                                                                                                                    \
      return ptl::add_layernorm<TYPE, float>(y, residual_out, residual_in, x, add_bias, w, b, rows, out_rows, hidden, eps, stream); \
    return ptl::add_layernorm<TYPE, TYPE>(y, residual_out, residual_in, x, add_bias, w, b, rows, out_rows, hidden, eps, stream);   \
  }                                                                                                                               \
  PTL_EXPORT int ptl_xielu##SUFFIX(void* out, const void* x, long long n, float ap, float aq, void* stream) {                      \
    return ptl::xielu<TYPE>(out, x, n, ap, aq, stream);                                                                           \
  }
PTL_LAYERNORM(_f32, float)
PTL_LAYERNORM(_bf16, __nv_bfloat16)
