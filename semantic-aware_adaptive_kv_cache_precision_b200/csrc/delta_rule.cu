// The delta-rule recurrence with a decay and a removal rate for every key channel.
//
// For each head, with a state S of dim x dim (rows: key channels, columns: value channels)
// that is carried from token to token in fp32:
//
//   w = exp(-decay_scale * sigmoid(w0 + W2 tanh(l)))      l: the low-rank projection's output
//   a = sigmoid(a_pre + a_bias)
//   u = k / sqrt(sum(k^2) + key_eps)
//   S <- diag(w) S - (a * u)(u^T S) + k v^T                 (both terms read the old S)
//   o = S^T r;   out = o / sqrt(mean(o^2) + eps) * norm_w * sigmoid(g)
//
// One block for each (head, sequence): thread j owns column j of S in registers and walks
// the sequence's tokens of this step in order; the per-channel numbers (r, k, w, u, a * u) of
// a token are worked out by the threads together and handed over through shared memory. The
// same kernel runs a prompt, a piece of one and a single decoded token, with the same sums
// in the same order, so a token's output does not depend on how the tokens came. r, k, v,
// g, a_pre and l are columns of one fp32 projection output [tokens, proj_stride].
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf(float z) { return 1.f / (1.f + expf(-z)); }

template <int DK, typename W, typename Out>
__global__ void __launch_bounds__(DK < 32 ? 32 : DK)
delta_rule_kernel(const float* __restrict__ proj, long long proj_stride, int off_r, int off_k,
                  int off_v, int off_g, int off_a, int off_l, const W* __restrict__ w2,
                  const W* __restrict__ w0, const W* __restrict__ a_bias,
                  const W* __restrict__ norm_w, float* __restrict__ state,
                  const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ slots,
                  Out* __restrict__ out, int heads, int dim, int rank, float decay_scale,
                  float key_eps, float eps, int keep_state) {
  extern __shared__ float shared[];
  float* s_l = shared;                 // [rank] tanh of the low-rank output
  float* s_w2 = s_l + rank;            // [dim, rank] this head's rows of W2
  __shared__ float s_r[DK], s_k[DK], s_w[DK], s_u[DK], s_b[DK];
  __shared__ float scratch[33];
  let_next_kernel_start();
  const int head = blockIdx.x, seq = blockIdx.y, tid = threadIdx.x;
  const int ch = head * dim + tid;
  const bool mine = tid < dim;
  for (int i = tid; i < dim * rank; i += blockDim.x)
    s_w2[i] = widen(w2[(long long)head * dim * rank + i]);
  const float my_w0 = mine ? widen(w0[ch]) : 0.f;
  const float my_ab = mine ? widen(a_bias[ch]) : 0.f;
  const float my_nw = mine ? widen(norm_w[ch]) : 0.f;
  wait_for_previous_kernel();
  const int begin = cu_seqlens[seq], end = cu_seqlens[seq + 1];
  float* my_state = state + (((long long)slots[seq] * heads + head) * dim) * dim + tid;
  float S[DK];
#pragma unroll
  for (int i = 0; i < DK; ++i) S[i] = (mine && i < dim) ? my_state[(long long)i * dim] : 0.f;
  __syncthreads();

  for (int t = begin; t < end; ++t) {
    const float* row = proj + (long long)t * proj_stride;
    for (int j = tid; j < rank; j += blockDim.x) s_l[j] = tanhf(row[off_l + j]);
    float k = 0.f, r = 0.f, a = 0.f, v = 0.f, g = 0.f;
    if (mine) {
      k = row[off_k + ch];
      r = row[off_r + ch];
      a = sigmoidf(row[off_a + ch] + my_ab);
      v = row[off_v + ch];
      g = row[off_g + ch];
    }
    const float kk = block_sum(k * k, scratch);      // (its barriers also publish s_l)
    if (mine) {
      float z = my_w0;
      const float* w2row = s_w2 + tid * rank;
      for (int j = 0; j < rank; ++j) z = fmaf(w2row[j], s_l[j], z);
      const float u = k / sqrtf(kk + key_eps);
      s_r[tid] = r;
      s_k[tid] = k;
      s_w[tid] = expf(-decay_scale * sigmoidf(z));
      s_u[tid] = u;
      s_b[tid] = a * u;
    }
    __syncthreads();
    float o = 0.f;
    if (mine) {
      float sa = 0.f;
#pragma unroll
      for (int i = 0; i < DK; ++i)
        if (i < dim) sa = fmaf(s_u[i], S[i], sa);
#pragma unroll
      for (int i = 0; i < DK; ++i)
        if (i < dim) {
          S[i] = fmaf(s_w[i], S[i], fmaf(-s_b[i], sa, s_k[i] * v));
          o = fmaf(S[i], s_r[i], o);
        }
    }
    const float oo = block_sum(o * o, scratch);
    if (mine)
      out[(long long)t * heads * dim + ch] =
          narrow<Out>(o / sqrtf(oo / (float)dim + eps) * my_nw * sigmoidf(g));
  }
  if (keep_state && mine) {
#pragma unroll
    for (int i = 0; i < DK; ++i)
      if (i < dim) my_state[(long long)i * dim] = S[i];
  }
}

template <int DK, typename W>
int launch(const float* proj, long long proj_stride, const int* off, const void* w2,
           const void* w0, const void* a_bias, const void* norm_w, float* state,
           const int32_t* cu_seqlens, const int32_t* slots, void* out, int out_dtype,
           int sequences, int heads, int dim, int rank, float decay_scale, float key_eps,
           float eps, int keep_state, cudaStream_t stream) {
  const size_t smem = ((size_t)rank + (size_t)dim * rank) * sizeof(float);
  if (smem > 160 * 1024) return cudaErrorInvalidValue;
  const int threads = ((dim + 31) / 32) * 32;
  auto go = [&](auto kernel, auto* o) {
    if (smem > 40 * 1024) {
      const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    return launch_overlapped(kernel, dim3(heads, sequences), dim3(threads), smem, stream, 1, proj,
                             proj_stride, off[0], off[1], off[2], off[3], off[4], off[5],
                             (const W*)w2, (const W*)w0, (const W*)a_bias, (const W*)norm_w, state,
                             cu_seqlens, slots, o, heads, dim, rank, decay_scale, key_eps, eps,
                             keep_state);
  };
  if (out_dtype == SAKV_F32) return go(delta_rule_kernel<DK, W, float>, (float*)out);
  if (out_dtype == SAKV_BF16)
    return go(delta_rule_kernel<DK, W, __nv_bfloat16>, (__nv_bfloat16*)out);
  return cudaErrorInvalidValue;
}

template <typename W>
int pick(int dim, const float* proj, long long proj_stride, const int* off, const void* w2,
         const void* w0, const void* a_bias, const void* norm_w, float* state,
         const int32_t* cu_seqlens, const int32_t* slots, void* out, int out_dtype, int sequences,
         int heads, int rank, float decay_scale, float key_eps, float eps, int keep_state,
         cudaStream_t stream) {
#define SAKV_DELTA(DK)                                                                          \
  return launch<DK, W>(proj, proj_stride, off, w2, w0, a_bias, norm_w, state, cu_seqlens, slots, \
                       out, out_dtype, sequences, heads, dim, rank, decay_scale, key_eps, eps,   \
                       keep_state, stream)
  if (dim <= 16) SAKV_DELTA(16);
  if (dim <= 32) SAKV_DELTA(32);
  if (dim <= 64) SAKV_DELTA(64);
  if (dim <= 128) SAKV_DELTA(128);
  SAKV_DELTA(256);
#undef SAKV_DELTA
}

}  // namespace

// proj: fp32 [tokens, proj_stride]; offsets[6]: the first column of r, k, v, g, a_pre (each
// heads * dim wide) and of l (rank wide). w2 [heads * dim, rank], w0, a_bias, norm_w
// [heads * dim] of type `w_dtype`. state: fp32 [slots, heads, dim, dim]. out: [tokens,
// heads * dim] of `out_dtype`. Sequence i of the step owns the tokens cu_seqlens[i] ..
// cu_seqlens[i + 1] - 1 and the state of slot slots[i].
SAKV_EXPORT int sakv_delta_rule(const float* proj, long long proj_stride, int off_r, int off_k,
                                int off_v, int off_g, int off_a, int off_l, const void* w2,
                                const void* w0, const void* a_bias, const void* norm_w,
                                int w_dtype, float* state, const int32_t* cu_seqlens,
                                const int32_t* slots, void* out, int out_dtype, int sequences,
                                int heads, int dim, int rank, float decay_scale, float key_eps,
                                float eps, int keep_state, cudaStream_t stream) {
  if (sequences < 0 || heads <= 0 || dim <= 0 || dim > 256 || rank <= 0 || sequences > 65535)
    return cudaErrorInvalidValue;
  if (sequences == 0) return 0;
  const int off[6] = {off_r, off_k, off_v, off_g, off_a, off_l};
  if (w_dtype == SAKV_F32)
    return pick<float>(dim, proj, proj_stride, off, w2, w0, a_bias, norm_w, state, cu_seqlens,
                       slots, out, out_dtype, sequences, heads, rank, decay_scale, key_eps, eps,
                       keep_state, stream);
  if (w_dtype == SAKV_BF16)
    return pick<__nv_bfloat16>(dim, proj, proj_stride, off, w2, w0, a_bias, norm_w, state,
                               cu_seqlens, slots, out, out_dtype, sequences, heads, rank,
                               decay_scale, key_eps, eps, keep_state, stream);
  return cudaErrorInvalidValue;
}
