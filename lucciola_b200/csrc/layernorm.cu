// Layer norm with a weight and no bias, y = (x - mean) / sqrt(var + eps) * w, var the mean of the squared
// deviations, everything in 32-bit; and the same norm on a sublayer's OUTPUT, fused with the scaled add into the
// residual stream, for blocks that norm what a sublayer returns instead of what it reads:
//
//   v        = sa * a [+ sb * b]              (a, b: outputs of one or two sublayers that ran side by side)
//   residual += mult * layernorm(v) * w
//   copy     = residual, rounded to the activation type (optional: what the next sublayer's products read)
//
// One CTA a row.  The mean is formed first and the variance from the deviations (two passes over a row that
// the first pass left in cache), so a row far from zero loses nothing.  The order of every sum is fixed by the
// row's length and the CTA's size, never by the batch.
#include "common.cuh"

namespace lb {

template <typename TO>
__global__ void layernorm_kernel(TO* __restrict__ out, const float* __restrict__ x, const float* __restrict__ weight,
                                 const int* __restrict__ rows, int hidden, float eps) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const int i = blockIdx.x;
  const float* r = x + (size_t)(rows ? rows[i] : i) * hidden;
  float s = 0.f;
  for (int j = threadIdx.x; j < hidden; j += blockDim.x) s += r[j];
  const float mean = block_sum(s, scratch) / (float)hidden;
  float ss = 0.f;
  for (int j = threadIdx.x; j < hidden; j += blockDim.x) { const float d = r[j] - mean; ss += d * d; }
  const float inv = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps);
  TO* o = out + (size_t)i * hidden;
  for (int j = threadIdx.x; j < hidden; j += blockDim.x) o[j] = from_f32<TO>((r[j] - mean) * inv * weight[j]);
}

template <typename TY, typename TC>
__global__ void layernorm_add_kernel(float* __restrict__ residual, const TY* __restrict__ a, const TY* __restrict__ b,
                                     float sa, float sb, const float* __restrict__ weight, float mult, float eps,
                                     TC* __restrict__ copy, int hidden) {
  __shared__ float scratch[33];
  pdl_trigger();
  pdl_wait();
  const size_t row = (size_t)blockIdx.x * hidden;
  const TY* ra = a + row;
  const TY* rb = b ? b + row : nullptr;
  auto value = [&](int j) { return rb ? fmaf(sb, to_f32(rb[j]), sa * to_f32(ra[j])) : sa * to_f32(ra[j]); };
  float s = 0.f;
  for (int j = threadIdx.x; j < hidden; j += blockDim.x) s += value(j);
  const float mean = block_sum(s, scratch) / (float)hidden;
  float ss = 0.f;
  for (int j = threadIdx.x; j < hidden; j += blockDim.x) { const float d = value(j) - mean; ss += d * d; }
  const float inv = rsqrtf(block_sum(ss, scratch) / (float)hidden + eps);
  float* r = residual + row;
  for (int j = threadIdx.x; j < hidden; j += blockDim.x) {
    const float v = fmaf(mult, (value(j) - mean) * inv * weight[j], r[j]);
    r[j] = v;
    if (copy) copy[row + j] = from_f32<TC>(v);
  }
}

template <typename TC>
__global__ void round_copy_kernel(TC* __restrict__ out, const float* __restrict__ x, long long n) {
  pdl_trigger();
  pdl_wait();
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    out[i] = from_f32<TC>(x[i]);
}

static int ln_threads(int hidden) { return hidden >= 4096 ? 512 : (hidden >= 1024 ? 256 : (hidden >= 256 ? 128 : 64)); }

}  // namespace lb

// out[i] = layernorm(x[rows ? rows[i] : i]) * weight; x float32 [*, hidden]
LB_EXPORT int lb_layernorm(void* out, int out_dtype, const float* x, const float* weight, const int* rows, int num_rows,
                           int hidden, float eps, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(out_dtype) && out && x && weight, "layernorm: bad arguments");
  LB_CHECK_ARG(num_rows >= 0 && hidden > 0, "layernorm: bad sizes rows=%d hidden=%d", num_rows, hidden);
  if (num_rows == 0) return 0;
  LB_DISPATCH_DTYPE(out_dtype, TO, {
    lb::launch(lb::layernorm_kernel<TO>, dim3(num_rows), dim3(lb::ln_threads(hidden)), 0, stream, (TO*)out, x, weight, rows, hidden, eps);
  })
  LB_CHECK_LAUNCH("layernorm");
  return 0;
}

// residual += mult * layernorm(sa * a [+ sb * b]) * weight; copy (optional, copy_dtype) = the new residual rounded.
// a, b: [num_rows, hidden] of y_dtype, contiguous.
LB_EXPORT int lb_layernorm_add(float* residual, const void* a, const void* b, int y_dtype, float sa, float sb,
                               const float* weight, float mult, float eps, void* copy, int copy_dtype, int num_rows,
                               int hidden, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(y_dtype) && lb::valid_dtype(copy_dtype) && residual && a && weight, "layernorm_add: bad arguments");
  LB_CHECK_ARG(num_rows >= 0 && hidden > 0, "layernorm_add: bad sizes rows=%d hidden=%d", num_rows, hidden);
  if (num_rows == 0) return 0;
  LB_DISPATCH_DTYPE(y_dtype, TY, {
    LB_DISPATCH_DTYPE(copy_dtype, TC, {
      lb::launch(lb::layernorm_add_kernel<TY, TC>, dim3(num_rows), dim3(lb::ln_threads(hidden)), 0, stream, residual, (const TY*)a,
                 (const TY*)b, sa, sb, weight, mult, eps, (TC*)copy, hidden);
    })
  })
  LB_CHECK_LAUNCH("layernorm_add");
  return 0;
}

// out = x rounded to out_dtype (the residual stream as the products of a sublayer read it)
LB_EXPORT int lb_round_copy(void* out, int out_dtype, const float* x, long long n, cudaStream_t stream) {
  LB_CHECK_ARG(lb::valid_dtype(out_dtype) && out && x && n >= 0, "round_copy: bad arguments");
  if (n == 0) return 0;
  long long blocks = (n + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  LB_DISPATCH_DTYPE(out_dtype, TC, {
    lb::launch(lb::round_copy_kernel<TC>, dim3((unsigned)blocks), dim3(256), 0, stream, (TC*)out, x, n);
  })
  LB_CHECK_LAUNCH("round_copy");
  return 0;
}
