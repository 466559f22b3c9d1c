// Layer norm with a weight and no bias over rows of the fp32 residual stream:
//   out = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w
// mean, deviations, variance and products in fp32, one rounding at the store. One block a
// row, the row kept in shared memory; the order of the additions depends on the row length
// alone, never on how many rows are in the batch.
//
// The second entry point is the step between two sublayers of a layer that norms a
// sublayer's OUTPUT as well as its input:
//   x += norm(y) * w_after;   out = norm(x) * w_before_next
// one pass over the stream instead of three (either half may be absent: without `y` it is
// the plain norm, without `w_before_next` only the stream is completed).
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

// (mean, 1 / sqrt(variance + eps)) of `row` (shared memory), every thread gets both
__device__ __forceinline__ float2 row_stats(const float* row, int hidden, float eps,
                                            float* scratch) {
  float s = 0.f;
  for (int i = threadIdx.x; i < hidden; i += kThreads) s += row[i];
  const float mean = block_sum(s, scratch) / static_cast<float>(hidden);
  float q = 0.f;
  for (int i = threadIdx.x; i < hidden; i += kThreads) {
    const float d = row[i] - mean;
    q = fmaf(d, d, q);
  }
  const float var = block_sum(q, scratch) / static_cast<float>(hidden);
  return make_float2(mean, rsqrtf(var + eps));
}

template <typename W, typename Out>
__global__ void __launch_bounds__(kThreads)
layer_norm_kernel(float* __restrict__ x, const float* __restrict__ y,
                  const W* __restrict__ w_after, const int32_t* __restrict__ rows,
                  const W* __restrict__ w_before, Out* __restrict__ out, int hidden, float eps) {
  extern __shared__ float row[];
  __shared__ float scratch[33];
  const long long src = rows ? rows[blockIdx.x] : blockIdx.x;
  float* in = x + src * hidden;
  if (y != nullptr) {
    const float* add = y + src * hidden;
    for (int i = threadIdx.x; i < hidden; i += kThreads) row[i] = add[i];
    __syncthreads();
    const float2 st = row_stats(row, hidden, eps, scratch);
    for (int i = threadIdx.x; i < hidden; i += kThreads) {
      const float v = in[i] + (row[i] - st.x) * st.y * widen(w_after[i]);
      in[i] = v;
      row[i] = v;
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += kThreads) row[i] = in[i];
  }
  if (out == nullptr) return;
  __syncthreads();
  const float2 st = row_stats(row, hidden, eps, scratch);
  Out* o = out + (long long)blockIdx.x * hidden;
  for (int i = threadIdx.x; i < hidden; i += kThreads)
    o[i] = narrow<Out>((row[i] - st.x) * st.y * widen(w_before[i]));
}

template <typename W, typename Out>
int launch(float* x, const float* y, const void* w_after, const int32_t* rows,
           const void* w_before, void* out, int n, int hidden, float eps, cudaStream_t stream) {
  return launch_ordered(layer_norm_kernel<W, Out>, dim3(n), dim3(kThreads),
                           (size_t)hidden * sizeof(float), stream, x, y, (const W*)w_after,
                           rows, (const W*)w_before, (Out*)out, hidden, eps);
}

}  // namespace

// x: fp32 [T, hidden], updated in place when `y` (fp32 [T, hidden]) is given: x += norm(y) *
// w_after. out (may be null): [n, hidden] = norm(x[rows ? rows[r] : r]) * w_before. `rows`
// only without `y`. Weights of `w_dtype`, out of `out_dtype`.
SAKV_EXPORT int sakv_layer_norm(float* x, const float* y, const void* w_after,
                                const int32_t* rows, const void* w_before, int w_dtype, void* out,
                                int out_dtype, int n, int hidden, float eps, cudaStream_t stream) {
  if (n < 0 || hidden <= 0 || hidden > 12000 || (y != nullptr && (rows != nullptr || !w_after)) ||
      (out != nullptr && !w_before) || (out == nullptr && y == nullptr))
    return cudaErrorInvalidValue;
  if (n == 0) return 0;
  if (w_dtype == SAKV_F32 && out_dtype == SAKV_F32)
    return launch<float, float>(x, y, w_after, rows, w_before, out, n, hidden, eps, stream);
  if (w_dtype == SAKV_BF16 && out_dtype == SAKV_BF16)
    return launch<__nv_bfloat16, __nv_bfloat16>(x, y, w_after, rows, w_before, out, n, hidden,
                                                eps, stream);
  if (w_dtype == SAKV_BF16 && out_dtype == SAKV_F32)
    return launch<__nv_bfloat16, float>(x, y, w_after, rows, w_before, out, n, hidden, eps, stream);
  if (w_dtype == SAKV_F32 && out_dtype == SAKV_BF16)
    return launch<float, __nv_bfloat16>(x, y, w_after, rows, w_before, out, n, hidden, eps, stream);
  return cudaErrorInvalidValue;
}
