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
// Three kernels. `delta_prepare` works out what does not depend on the state, for all tokens
// side by side (a warp a token and head): w, u and a * u, fp32 [tokens, 3, heads * dim].
// `delta_scan` is the recurrence: a block has some neighbouring columns of one head's state
// for one sequence (columns never meet, so a head may be spread over several blocks when
// there are few heads and sequences) and walks the sequence's tokens of this step in chunks
// whose r, k, v, w, u, a * u are copied into shared memory one chunk ahead (cp.async, two
// buffers). The state is in registers: a column's rows are dealt to R neighbouring lanes, and
// the two sums over a column (u^T S and S^T r) are finished with shuffles among them.
// Block-wide barriers are paid per chunk, not per token. `delta_finish` norms and gates the
// raw outputs, a warp a token and head. The same kernels run a prompt, a piece of one and a
// single decoded token,
// and every sum has the same terms in the same order however the tokens are cut into steps
// and chunks, so a token's output does not depend on how the tokens came. r, k, v, g, a_pre
// and l are columns of one fp32 projection output [tokens, proj_stride].
#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoidf(float z) { return 1.f / (1.f + expf(-z)); }

constexpr int kPrepareTokens = 8;      // tokens (warps) of a block of `delta_prepare`

template <typename W>
__global__ void __launch_bounds__(kPrepareTokens * 32)
delta_prepare_kernel(const float* __restrict__ proj, long long proj_stride, int off_k, int off_a,
                     int off_l, const W* __restrict__ w2, const W* __restrict__ w0,
                     const W* __restrict__ a_bias, float* __restrict__ prepared, int tokens,
                     int heads, int dim, int rank, float decay_scale, float key_eps) {
  extern __shared__ float shared[];
  const int ld2 = rank + 1;                         // padded rows of W2: no bank conflicts
  float* s_w2 = shared;                             // [dim][rank + 1]
  float* s_l = s_w2 + dim * ld2;                    // [warps][rank]
  let_next_kernel_start();
  const int head = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int base = head * dim;
  for (int i = threadIdx.x; i < dim * rank; i += blockDim.x)
    s_w2[(i / rank) * ld2 + i % rank] = widen(w2[(long long)base * rank + i]);
  wait_for_previous_kernel();
  const long long t = (long long)blockIdx.x * kPrepareTokens + warp;
  const bool live = t < tokens;
  const float* row = proj + (live ? t : 0) * proj_stride;
  float* l = s_l + warp * rank;
  for (int j = lane; j < rank; j += 32) l[j] = tanhf(row[off_l + j]);
  __syncthreads();
  if (!live) return;
  float kk = 0.f;
  for (int c = lane; c < dim; c += 32) {
    const float k = row[off_k + base + c];
    kk = fmaf(k, k, kk);
  }
  const float inv = 1.f / sqrtf(warp_sum(kk) + key_eps);
  const long long hd = (long long)heads * dim;
  float* dst = prepared + t * 3 * hd + base;
  for (int c = lane; c < dim; c += 32) {
    float z = widen(w0[base + c]);
    const float* w2row = s_w2 + c * ld2;
    for (int j = 0; j < rank; ++j) z = fmaf(w2row[j], l[j], z);
    const float u = row[off_k + base + c] * inv;
    dst[c] = expf(-decay_scale * sigmoidf(z));
    dst[hd + c] = u;
    dst[2 * hd + c] = sigmoidf(row[off_a + base + c] + widen(a_bias[base + c])) * u;
  }
}

template <int R>
__device__ __forceinline__ float sum_over_parts(float v) {
#pragma unroll
  for (int o = 1; o < R; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ void copy16_async(float* dst, const float* src) {
  const uint32_t to = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(to), "l"(src) : "memory");
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void copies_wait_all_but_last() {
  asm volatile("cp.async.wait_group 1;" ::: "memory");
}

// One block: `cols` neighbouring columns of one head's state for one sequence. A column's
// rows are dealt to R neighbouring lanes, dim / R <= RPT rows each. VEC: rows are read four
// at a time (dim / R a multiple of 4, everything 16-byte aligned). The raw o = S^T r goes to
// `raw` [tokens, heads * dim] fp32 for `delta_finish`.
template <int RPT, int R, bool VEC>
__global__ void __launch_bounds__(512)
delta_scan_kernel(const float* __restrict__ proj, long long proj_stride, int off_r, int off_k,
                  int off_v, const float* __restrict__ prepared, float* __restrict__ state,
                  const int32_t* __restrict__ cu_seqlens, const int32_t* __restrict__ slots,
                  float* __restrict__ raw, int heads, int dim, int cols, int chunk,
                  int keep_state) {
  extern __shared__ __align__(16) float shared[];
  // a token's per-row vectors lie part by part with four floats between the parts, so that the
  // R lanes of a column read from different banks
  const int rpt = dim / R;
  const int ldp = rpt + (R > 1 ? 4 : 0), ldt = R * ldp;      // a part's, a token's stride
  const int per_buffer = chunk * (5 * ldt + cols);
  let_next_kernel_start();
  const int head = blockIdx.x, seq = blockIdx.y, col0 = blockIdx.z * cols;
  const int tid = threadIdx.x, threads = blockDim.x;
  const int mycol = tid / R, part = tid % R, col = col0 + mycol;
  const bool mine = mycol < cols && col < dim;
  const int base = head * dim;
  const long long hd = (long long)heads * dim;
  wait_for_previous_kernel();
  const int begin = cu_seqlens[seq], end = cu_seqlens[seq + 1];
  float* my_state = state + (((long long)slots[seq] * heads + head) * dim + part * rpt) * dim + col;
  float S[RPT];
#pragma unroll
  for (int i = 0; i < RPT; ++i) S[i] = (mine && i < rpt) ? my_state[(long long)i * dim] : 0.f;

  const bool aligned = VEC && dim % 4 == 0 && cols % 4 == 0 && proj_stride % 4 == 0 &&
                       off_r % 4 == 0 && off_k % 4 == 0 && off_v % 4 == 0 &&
                       !((uintptr_t)proj & 15) && !((uintptr_t)prepared & 15);
  // the rows of a chunk: r, k (from proj) and w, u, a*u (prepared), part by part; then this
  // block's columns of v
  auto fetch = [&](int t0, int buffer) {
    const int count = min(chunk, end - t0);
    float* dst = shared + buffer * per_buffer;
    float* dst_v = dst + chunk * 5 * ldt;
    // (an item is four floats, or one, of one of the six vectors; its place in the token is
    // worked out once, then it is copied for every token of the chunk)
    if (aligned) {
      const int quads = dim / 4, vquads = cols / 4, per_token = 5 * quads + vquads;
      for (int j = tid; j < per_token; j += threads) {
        const float* src;
        float* to;
        long long src_step = proj_stride;
        int to_step = 5 * ldt;
        if (j >= 5 * quads) {
          const int c = (j - 5 * quads) * 4;
          src = proj + (long long)t0 * proj_stride + off_v + base + col0 + c;
          to = dst_v + c;
          to_step = cols;
        } else {
          const int which = j / quads, c = (j - which * quads) * 4;
          to = dst + which * ldt + (c / rpt) * ldp + c % rpt;
          if (which < 2) {
            src = proj + (long long)t0 * proj_stride + (which == 0 ? off_r : off_k) + base + c;
          } else {
            src = prepared + ((long long)t0 * 3 + (which - 2)) * hd + base + c;
            src_step = 3 * hd;
          }
        }
        for (int tt = 0; tt < count; ++tt) copy16_async(to + tt * to_step, src + tt * src_step);
      }
    } else {
      const int per_token = 5 * dim + cols;
      for (int j = tid; j < per_token; j += threads) {
        const float* src;
        float* to;
        long long src_step = proj_stride;
        int to_step = 5 * ldt;
        bool real = true;
        if (j >= 5 * dim) {
          const int c = j - 5 * dim;
          real = col0 + c < dim;
          src = proj + (long long)t0 * proj_stride + off_v + base + col0 + c;
          to = dst_v + c;
          to_step = cols;
        } else {
          const int which = j / dim, c = j - which * dim;
          to = dst + which * ldt + (c / rpt) * ldp + c % rpt;
          if (which < 2) {
            src = proj + (long long)t0 * proj_stride + (which == 0 ? off_r : off_k) + base + c;
          } else {
            src = prepared + ((long long)t0 * 3 + (which - 2)) * hd + base + c;
            src_step = 3 * hd;
          }
        }
        for (int tt = 0; tt < count; ++tt) to[tt * to_step] = real ? src[tt * src_step] : 0.f;
      }
    }
    copies_commit();
  };

  int buffer = 0;
  if (begin < end) fetch(begin, 0);
  for (int t0 = begin; t0 < end; t0 += chunk, buffer ^= 1) {
    const int count = min(chunk, end - t0);
    if (t0 + chunk < end) fetch(t0 + chunk, buffer ^ 1);
    else copies_commit();
    copies_wait_all_but_last();
    __syncthreads();                                 // the chunk has landed, for everyone
    const float* rows = shared + buffer * per_buffer + part * ldp;
    const float* vals = shared + buffer * per_buffer + chunk * 5 * ldt + (mine ? mycol : 0);
    for (int tt = 0; tt < count; ++tt) {             // the recurrence
      const float* x = rows + tt * 5 * ldt;          // r, k, w, u, a*u: ldt apart
      const float v = vals[tt * cols];
      float sa = 0.f, o = 0.f;
      if constexpr (VEC) {
        float r[RPT], k[RPT], w[RPT], u[RPT], b[RPT];
#pragma unroll
        for (int i = 0; i < RPT; i += 4)
          if (i < rpt) {
            *reinterpret_cast<float4*>(u + i) = *reinterpret_cast<const float4*>(x + 3 * ldt + i);
            *reinterpret_cast<float4*>(r + i) = *reinterpret_cast<const float4*>(x + i);
            *reinterpret_cast<float4*>(k + i) = *reinterpret_cast<const float4*>(x + ldt + i);
            *reinterpret_cast<float4*>(w + i) = *reinterpret_cast<const float4*>(x + 2 * ldt + i);
            *reinterpret_cast<float4*>(b + i) = *reinterpret_cast<const float4*>(x + 4 * ldt + i);
          }
#pragma unroll
        for (int i = 0; i < RPT; ++i)
          if (i < rpt) sa = fmaf(u[i], S[i], sa);
        sa = sum_over_parts<R>(sa);
#pragma unroll
        for (int i = 0; i < RPT; ++i)
          if (i < rpt) {
            S[i] = fmaf(w[i], S[i], fmaf(-b[i], sa, k[i] * v));
            o = fmaf(S[i], r[i], o);
          }
      } else {
#pragma unroll
        for (int i = 0; i < RPT; ++i)
          if (i < rpt) sa = fmaf(x[3 * ldt + i], S[i], sa);
        sa = sum_over_parts<R>(sa);
#pragma unroll
        for (int i = 0; i < RPT; ++i)
          if (i < rpt) {
            S[i] = fmaf(x[2 * ldt + i], S[i], fmaf(-x[4 * ldt + i], sa, x[ldt + i] * v));
            o = fmaf(S[i], x[i], o);
          }
      }
      o = sum_over_parts<R>(o);
      if (mine && part == 0) raw[(long long)(t0 + tt) * hd + base + col] = o;
    }
    __syncthreads();                                 // everyone is done with this buffer
  }
  if (keep_state && mine) {
#pragma unroll
    for (int i = 0; i < RPT; ++i)
      if (i < rpt) my_state[(long long)i * dim] = S[i];
  }
}

// out = raw / sqrt(mean(raw^2) + eps) * norm_w * sigmoid(g), head by head: a warp for each
// (token, head).
template <typename W, typename Out>
__global__ void delta_finish_kernel(const float* __restrict__ raw, const float* __restrict__ proj,
                                    long long proj_stride, int off_g,
                                    const W* __restrict__ norm_w, Out* __restrict__ out,
                                    long long items, int heads, int dim, float eps) {
  let_next_kernel_start();
  wait_for_previous_kernel();
  const long long item = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (item >= items) return;
  const long long t = item / heads;
  const int base = static_cast<int>(item - t * heads) * dim;
  const float* o = raw + t * heads * dim + base;
  float oo = 0.f;
  for (int c = lane; c < dim; c += 32) oo = fmaf(o[c], o[c], oo);
  const float inv = 1.f / sqrtf(warp_sum(oo) / (float)dim + eps);
  for (int c = lane; c < dim; c += 32)
    out[t * heads * dim + base + c] = narrow<Out>(
        o[c] * inv * widen(norm_w[base + c]) * sigmoidf(proj[t * proj_stride + off_g + base + c]));
}

constexpr size_t kScanBudget = 96 * 1024;

template <int RPT, int R, bool VEC>
int launch_scan(const float* proj, long long proj_stride, const int* off, const float* prepared,
                float* state, const int32_t* cu_seqlens, const int32_t* slots, float* raw,
                int sequences, int heads, int dim, int chunk, int keep_state,
                cudaStream_t stream) {
  // columns a block: few enough that the blocks fill the GPU, at least 128 threads' worth
  int cols = dim;
  if (VEC) {
    const int least = 128 / R > 4 ? 128 / R : 4;
    while (cols % 8 == 0 && cols / 2 >= least &&
           (long long)heads * sequences * (dim / cols) * 2 <= sm_count() * 2)
      cols /= 2;
    while (cols * R > 512 && cols % 8 == 0) cols /= 2;
  }
  if (cols * R > 512) return cudaErrorInvalidValue;
  const int rpt = dim / R, ldt = R * (rpt + (R > 1 ? 4 : 0));
  auto bytes = [&](int n) { return (size_t)2 * n * (5 * ldt + cols) * sizeof(float); };
  if (chunk < 1) chunk = 1;
  if (chunk > 16) chunk = 16;
  while (chunk > 1 && bytes(chunk) > kScanBudget) chunk /= 2;
  if (bytes(chunk) > kScanBudget) return cudaErrorInvalidValue;
  const int threads = ((cols * R + 31) / 32) * 32;
  static PerDeviceOnce configured;
  auto kernel = delta_scan_kernel<RPT, R, VEC>;
  if (configured.needs()) {
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)kScanBudget);
    if (e != cudaSuccess) return (int)e;
    configured.done();
  }
  return launch_overlapped(kernel, dim3(heads, sequences, (dim + cols - 1) / cols), dim3(threads),
                           bytes(chunk), stream, 1, proj, proj_stride, off[0], off[1], off[2],
                           prepared, state, cu_seqlens, slots, raw, heads, dim, cols, chunk,
                           keep_state);
}

int pick_scan(const float* proj, long long proj_stride, const int* off, const float* prepared,
              float* state, const int32_t* cu_seqlens, const int32_t* slots, float* raw,
              int sequences, int heads, int dim, int chunk, int keep_state, cudaStream_t stream) {
#define SAKV_SCAN(RPT, R, VEC)                                                                  \
  return launch_scan<RPT, R, VEC>(proj, proj_stride, off, prepared, state, cu_seqlens, slots,   \
                                  raw, sequences, heads, dim, chunk, keep_state, stream)
  // a column's rows over R lanes, four rows at a time: the most lanes (up to 16) that leave
  // a lane 8 rows, or 4 where dim is small; dims that 16 does not divide: one lane a column
  if (dim % 16 == 0) {
    int lanes = 4;
    while (lanes < 16 && dim % (8 * lanes) == 0 && dim / (2 * lanes) >= 8) lanes *= 2;
    const int rpt = dim / lanes;
    if (lanes == 4 && rpt <= 4) SAKV_SCAN(4, 4, true);
    if (lanes == 4 && rpt <= 8) SAKV_SCAN(8, 4, true);
    if (lanes == 4 && rpt <= 16) SAKV_SCAN(16, 4, true);
    if (lanes == 8 && rpt <= 8) SAKV_SCAN(8, 8, true);
    if (lanes == 8 && rpt <= 16) SAKV_SCAN(16, 8, true);
    if (lanes == 16 && rpt <= 8) SAKV_SCAN(8, 16, true);
    if (lanes == 16 && rpt <= 16) SAKV_SCAN(16, 16, true);
  }
  if (dim <= 32) SAKV_SCAN(32, 1, false);
  if (dim <= 64) SAKV_SCAN(64, 1, false);
  if (dim <= 128) SAKV_SCAN(128, 1, false);
  SAKV_SCAN(256, 1, false);
#undef SAKV_SCAN
}

template <typename W>
int run(const float* proj, long long proj_stride, const int* off, const void* w2, const void* w0,
        const void* a_bias, const void* norm_w, float* prepared, float* raw, float* state,
        const int32_t* cu_seqlens, const int32_t* slots, void* out, int out_dtype, int tokens,
        int sequences, int heads, int dim, int rank, int chunk, float decay_scale, float key_eps,
        float eps, int keep_state, cudaStream_t stream) {
  constexpr size_t kPrepareBudget = 200 * 1024;
  const size_t smem = ((size_t)dim * (rank + 1) + (size_t)kPrepareTokens * rank) * sizeof(float);
  if (smem > kPrepareBudget) return cudaErrorInvalidValue;
  static PerDeviceOnce configured;
  if (configured.needs()) {
    const cudaError_t e = cudaFuncSetAttribute(delta_prepare_kernel<W>,
                                               cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               (int)kPrepareBudget);
    if (e != cudaSuccess) return (int)e;
    configured.done();
  }
  int code = launch_overlapped(
      delta_prepare_kernel<W>, dim3((tokens + kPrepareTokens - 1) / kPrepareTokens, heads),
      dim3(kPrepareTokens * 32), smem, stream, 1, proj, proj_stride, off[1], off[4], off[5],
      (const W*)w2, (const W*)w0, (const W*)a_bias, prepared, tokens, heads, dim, rank,
      decay_scale, key_eps);
  if (code != 0) return code;
  code = pick_scan(proj, proj_stride, off, prepared, state, cu_seqlens, slots, raw, sequences,
                   heads, dim, chunk, keep_state, stream);
  if (code != 0) return code;
  const long long items = (long long)tokens * heads;
  const long long blocks = (items * 32 + 255) / 256;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
  if (out_dtype == SAKV_F32)
    return launch_overlapped(delta_finish_kernel<W, float>, dim3((unsigned)blocks), dim3(256), 0,
                             stream, 1, (const float*)raw, proj, proj_stride, off[3],
                             (const W*)norm_w, (float*)out, items, heads, dim, eps);
  if (out_dtype == SAKV_BF16)
    return launch_overlapped(delta_finish_kernel<W, __nv_bfloat16>, dim3((unsigned)blocks),
                             dim3(256), 0, stream, 1, (const float*)raw, proj, proj_stride, off[3],
                             (const W*)norm_w, (__nv_bfloat16*)out, items, heads, dim, eps);
  return cudaErrorInvalidValue;
}

}  // namespace

// proj: fp32 [tokens, proj_stride]; the first columns of r, k, v, g, a_pre (each heads * dim
// wide) and of l (rank wide) are given. w2 [heads * dim, rank], w0, a_bias, norm_w [heads *
// dim] of type `w_dtype`. prepared, raw: fp32 scratch [tokens, 3, heads * dim] and [tokens,
// heads * dim]. state: fp32 [slots,
// heads, dim, dim]. out: [tokens, heads * dim] of `out_dtype`. Sequence i of the step owns the
// tokens cu_seqlens[i] .. cu_seqlens[i + 1] - 1 and the state of slot slots[i]. `chunk`: how
// many tokens a block takes into shared memory at a time (the most a sequence brings in this
// step is enough; at most 16).
SAKV_EXPORT int sakv_delta_rule(const float* proj, long long proj_stride, int off_r, int off_k,
                                int off_v, int off_g, int off_a, int off_l, const void* w2,
                                const void* w0, const void* a_bias, const void* norm_w,
                                int w_dtype, float* prepared, float* raw, float* state,
                                const int32_t* cu_seqlens, const int32_t* slots, void* out,
                                int out_dtype, int tokens, int sequences, int heads, int dim,
                                int rank, int chunk, float decay_scale, float key_eps, float eps,
                                int keep_state, cudaStream_t stream) {
  if (tokens < 0 || sequences < 0 || heads <= 0 || heads > 65535 || dim <= 0 || dim > 256 ||
      rank <= 0 || sequences > 65535)
    return cudaErrorInvalidValue;
  if (sequences == 0 || tokens == 0) return 0;
  const int off[6] = {off_r, off_k, off_v, off_g, off_a, off_l};
  if (w_dtype == SAKV_F32)
    return run<float>(proj, proj_stride, off, w2, w0, a_bias, norm_w, prepared, raw, state,
                      cu_seqlens, slots, out, out_dtype, tokens, sequences, heads, dim, rank, chunk,
                      decay_scale, key_eps, eps, keep_state, stream);
  if (w_dtype == SAKV_BF16)
    return run<__nv_bfloat16>(proj, proj_stride, off, w2, w0, a_bias, norm_w, prepared, raw,
                              state, cu_seqlens, slots, out, out_dtype, tokens, sequences, heads, dim,
                              rank, chunk, decay_scale, key_eps, eps, keep_state, stream);
  return cudaErrorInvalidValue;
}
