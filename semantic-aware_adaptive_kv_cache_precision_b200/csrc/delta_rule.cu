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
// One block for each (head, sequence) walks the sequence's tokens of this step in chunks. For
// a chunk, all threads first work out the per-channel numbers of its tokens side by side (the
// decay's second matrix times tanh(l), the exponentials and sigmoids, the unit keys) and put
// them into shared memory; then the recurrence runs over the chunk's tokens with the state in
// registers: column j of S belongs to R neighbouring lanes, each with dim / R of its rows, and
// the two sums over a column (u^T S and S^T r) are finished with shuffles among them; then the
// chunk's outputs are normed and gated, a warp a token. Block-wide barriers are paid per
// chunk, not per token. The same kernel runs a prompt, a piece of one and a single decoded
// token, and every sum has the same terms in the same order however the tokens are cut into
// steps and chunks, so a token's output does not depend on how the tokens came. r, k, v, g,
// a_pre and l are columns of one fp32 projection output [tokens, proj_stride].
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf(float z) { return 1.f / (1.f + expf(-z)); }

template <int R>
__device__ __forceinline__ float sum_over_parts(float v) {
#pragma unroll
  for (int o = 1; o < R; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// RPT: the most rows of a column that one lane holds (dim / R <= RPT).
template <int RPT, int R, typename W, typename Out>
__global__ void __launch_bounds__(RPT * R * R < 32 ? 32 : RPT * R * R)
delta_rule_kernel(const float* __restrict__ proj, long long proj_stride, int off_r, int off_k,
                  int off_v, int off_g, int off_a, int off_l, const W* __restrict__ w2,
                  const W* __restrict__ w0, const W* __restrict__ a_bias,
                  const W* __restrict__ norm_w, float* __restrict__ state,
                  const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ slots,
                  Out* __restrict__ out, int heads, int dim, int rank, int chunk,
                  float decay_scale, float key_eps, float eps, int keep_state) {
  extern __shared__ float shared[];
  const int ld2 = rank + 1;                         // padded rows of W2: no bank conflicts
  float* s_w2 = shared;                             // [dim][rank + 1]
  float* s_w0 = s_w2 + dim * ld2;                   // [dim] each
  float* s_ab = s_w0 + dim;
  float* s_nw = s_ab + dim;
  float* s_l = s_nw + dim;                          // [chunk][rank]
  float* s_r = s_l + chunk * rank;                  // [chunk][dim] each
  float* s_k = s_r + chunk * dim;
  float* s_v = s_k + chunk * dim;
  float* s_w = s_v + chunk * dim;
  float* s_u = s_w + chunk * dim;
  float* s_b = s_u + chunk * dim;
  float* s_o = s_b + chunk * dim;
  let_next_kernel_start();
  const int head = blockIdx.x, seq = blockIdx.y, tid = threadIdx.x, threads = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5, warps = threads >> 5;
  const int rpt = dim / R;                          // rows a lane (R divides dim)
  const int col = tid / R, part = tid % R, row0 = part * rpt;
  const bool mine = col < dim;
  const int base = head * dim;
  for (int i = tid; i < dim * rank; i += threads)
    s_w2[(i / rank) * ld2 + i % rank] = widen(w2[(long long)base * rank + i]);
  for (int i = tid; i < dim; i += threads) {
    s_w0[i] = widen(w0[base + i]);
    s_ab[i] = widen(a_bias[base + i]);
    s_nw[i] = widen(norm_w[base + i]);
  }
  wait_for_previous_kernel();
  const int begin = cu_seqlens[seq], end = cu_seqlens[seq + 1];
  float* my_state = state + (((long long)slots[seq] * heads + head) * dim + row0) * dim + col;
  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) S[i] = (mine && i < rpt) ? my_state[(long long)i * dim] : 0.f;

  for (int t0 = begin; t0 < end; t0 += chunk) {
    const int count = min(chunk, end - t0);
    __syncthreads();                                // the chunk before is done with shared memory
    for (int i = tid; i < count * rank; i += threads) {
      const int tt = i / rank;
      s_l[i] = tanhf(proj[(long long)(t0 + tt) * proj_stride + off_l + (i - tt * rank)]);
    }
    __syncthreads();
    for (int i = tid; i < count * dim; i += threads) {
      const int tt = i / dim, c = i - tt * dim;
      const float* row = proj + (long long)(t0 + tt) * proj_stride + base + c;
      s_r[i] = row[off_r];
      s_k[i] = row[off_k];
      s_v[i] = row[off_v];
      float z = s_w0[c];
      const float* w2row = s_w2 + c * ld2;
      const float* l = s_l + tt * rank;
      for (int j = 0; j < rank; ++j) z = fmaf(w2row[j], l[j], z);
      s_w[i] = expf(-decay_scale * sigmoidf(z));
      s_b[i] = sigmoidf(row[off_a] + s_ab[c]);      // the removal rate, for now
    }
    __syncthreads();
    for (int tt = warp; tt < count; tt += warps) {  // unit keys: a warp a token
      float kk = 0.f;
      for (int c = lane; c < dim; c += 32) kk = fmaf(s_k[tt * dim + c], s_k[tt * dim + c], kk);
      const float inv = 1.f / sqrtf(warp_sum(kk) + key_eps);
      for (int c = lane; c < dim; c += 32) {
        const float u = s_k[tt * dim + c] * inv;
        s_u[tt * dim + c] = u;
        s_b[tt * dim + c] *= u;
      }
    }
    __syncthreads();
    for (int tt = 0; tt < count; ++tt) {            // the recurrence
      const int at = tt * dim + row0;
      float sa = 0.f, sa2 = 0.f;
#pragma unroll
      for (int i = 0; i < RPT; i += 2) {
        if (i < rpt) sa = fmaf(s_u[at + i], S[i], sa);
        if (i + 1 < rpt) sa2 = fmaf(s_u[at + i + 1], S[i + 1], sa2);
      }
      sa = sum_over_parts<R>(sa + sa2);
      const float v = mine ? s_v[tt * dim + col] : 0.f;
      float o = 0.f, o2 = 0.f;
#pragma unroll
      for (int i = 0; i < RPT; i += 2) {
        if (i < rpt) {
          S[i] = fmaf(s_w[at + i], S[i], fmaf(-s_b[at + i], sa, s_k[at + i] * v));
          o = fmaf(S[i], s_r[at + i], o);
        }
        if (i + 1 < rpt) {
          S[i + 1] = fmaf(s_w[at + i + 1], S[i + 1],
                          fmaf(-s_b[at + i + 1], sa, s_k[at + i + 1] * v));
          o2 = fmaf(S[i + 1], s_r[at + i + 1], o2);
        }
      }
      o = sum_over_parts<R>(o + o2);
      if (mine && part == 0) s_o[tt * dim + col] = o;
    }
    __syncthreads();
    for (int tt = warp; tt < count; tt += warps) {  // per-head norm and gate: a warp a token
      float oo = 0.f;
      for (int c = lane; c < dim; c += 32) oo = fmaf(s_o[tt * dim + c], s_o[tt * dim + c], oo);
      const float inv = 1.f / sqrtf(warp_sum(oo) / (float)dim + eps);
      const long long t = t0 + tt;
      for (int c = lane; c < dim; c += 32)
        out[t * heads * dim + base + c] =
            narrow<Out>(s_o[tt * dim + c] * inv * s_nw[c] *
                        sigmoidf(proj[t * proj_stride + off_g + base + c]));
    }
  }
  if (keep_state && mine) {
#pragma unroll
    for (int i = 0; i < RPT; ++i)
      if (i < rpt) my_state[(long long)i * dim] = S[i];
  }
}

size_t shared_bytes(int dim, int rank, int chunk) {
  return ((size_t)dim * (rank + 1) + 3 * (size_t)dim + (size_t)chunk * rank +
          7 * (size_t)chunk * dim) * sizeof(float);
}

template <int RPT, int R, typename W>
int launch(const float* proj, long long proj_stride, const int* off, const void* w2,
           const void* w0, const void* a_bias, const void* norm_w, float* state,
           const int32_t* cu_seqlens, const int32_t* slots, void* out, int out_dtype,
           int sequences, int heads, int dim, int rank, int chunk, float decay_scale,
           float key_eps, float eps, int keep_state, cudaStream_t stream) {
  constexpr size_t kBudget = 200 * 1024;
  if (chunk < 1) chunk = 1;
  if (chunk > 64) chunk = 64;
  while (chunk > 1 && shared_bytes(dim, rank, chunk) > kBudget / 2) chunk = (chunk + 1) / 2;
  const size_t smem = shared_bytes(dim, rank, chunk);
  if (smem > kBudget) return cudaErrorInvalidValue;
  const int threads = ((dim * R + 31) / 32) * 32;
  static PerDeviceOnce configured[2];
  auto go = [&](auto kernel, auto* o) {
    PerDeviceOnce& once = configured[out_dtype == SAKV_F32 ? 0 : 1];
    if (once.needs()) {
      const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)kBudget);
      if (e != cudaSuccess) return (int)e;
      once.done();
    }
    return launch_overlapped(kernel, dim3(heads, sequences), dim3(threads), smem, stream, 1, proj,
                             proj_stride, off[0], off[1], off[2], off[3], off[4], off[5],
                             (const W*)w2, (const W*)w0, (const W*)a_bias, (const W*)norm_w, state,
                             cu_seqlens, slots, o, heads, dim, rank, chunk, decay_scale, key_eps,
                             eps, keep_state);
  };
  if (out_dtype == SAKV_F32) return go(delta_rule_kernel<RPT, R, W, float>, (float*)out);
  if (out_dtype == SAKV_BF16)
    return go(delta_rule_kernel<RPT, R, W, __nv_bfloat16>, (__nv_bfloat16*)out);
  return cudaErrorInvalidValue;
}

template <typename W>
int pick(int dim, const float* proj, long long proj_stride, const int* off, const void* w2,
         const void* w0, const void* a_bias, const void* norm_w, float* state,
         const int32_t* cu_seqlens, const int32_t* slots, void* out, int out_dtype, int sequences,
         int heads, int rank, int chunk, float decay_scale, float key_eps, float eps,
         int keep_state, cudaStream_t stream) {
#define SAKV_DELTA(RPT, R)                                                                      \
  return launch<RPT, R, W>(proj, proj_stride, off, w2, w0, a_bias, norm_w, state, cu_seqlens,    \
                           slots, out, out_dtype, sequences, heads, dim, rank, chunk,            \
                           decay_scale, key_eps, eps, keep_state, stream)
  // a column's rows over 4 lanes where 4 divides dim, else over 2, else one lane a column
  if (dim % 4 == 0) {
    if (dim <= 32) SAKV_DELTA(8, 4);
    if (dim <= 64) SAKV_DELTA(16, 4);
    if (dim <= 128) SAKV_DELTA(32, 4);
    SAKV_DELTA(64, 4);
  }
  if (dim % 2 == 0) {
    if (dim <= 32) SAKV_DELTA(16, 2);
    if (dim <= 64) SAKV_DELTA(32, 2);
    if (dim <= 128) SAKV_DELTA(64, 2);
    SAKV_DELTA(128, 2);
  }
  if (dim <= 32) SAKV_DELTA(32, 1);
  if (dim <= 64) SAKV_DELTA(64, 1);
  if (dim <= 128) SAKV_DELTA(128, 1);
  SAKV_DELTA(256, 1);
#undef SAKV_DELTA
}

}  // namespace

// proj: fp32 [tokens, proj_stride]; offsets[6]: the first column of r, k, v, g, a_pre (each
// heads * dim wide) and of l (rank wide). w2 [heads * dim, rank], w0, a_bias, norm_w
// [heads * dim] of type `w_dtype`. state: fp32 [slots, heads, dim, dim]. out: [tokens,
// heads * dim] of `out_dtype`. Sequence i of the step owns the tokens cu_seqlens[i] ..
// cu_seqlens[i + 1] - 1 and the state of slot slots[i]. `chunk`: how many tokens a block takes
// into shared memory at a time (the most a sequence brings in this step is enough; at most 64).
SAKV_EXPORT int sakv_delta_rule(const float* proj, long long proj_stride, int off_r, int off_k,
                                int off_v, int off_g, int off_a, int off_l, const void* w2,
                                const void* w0, const void* a_bias, const void* norm_w,
                                int w_dtype, float* state, const int32_t* cu_seqlens,
                                const int32_t* slots, void* out, int out_dtype, int sequences,
                                int heads, int dim, int rank, int chunk, float decay_scale,
                                float key_eps, float eps, int keep_state, cudaStream_t stream) {
  if (sequences < 0 || heads <= 0 || dim <= 0 || dim > 256 || rank <= 0 || sequences > 65535)
    return cudaErrorInvalidValue;
  if (sequences == 0) return 0;
  const int off[6] = {off_r, off_k, off_v, off_g, off_a, off_l};
  if (w_dtype == SAKV_F32)
    return pick<float>(dim, proj, proj_stride, off, w2, w0, a_bias, norm_w, state, cu_seqlens,
                       slots, out, out_dtype, sequences, heads, rank, chunk, decay_scale, key_eps,
                       eps, keep_state, stream);
  if (w_dtype == SAKV_BF16)
    return pick<__nv_bfloat16>(dim, proj, proj_stride, off, w2, w0, a_bias, norm_w, state,
                               cu_seqlens, slots, out, out_dtype, sequences, heads, rank, chunk,
                               decay_scale, key_eps, eps, keep_state, stream);
  return cudaErrorInvalidValue;
}
