// Several copies of the residual stream ("streams") and what a layer does with them.
//
// A sublayer reads a weighted sum of the streams and writes its output back to all of them:
//
//   u   = sum_s in[s] x_s                          (then RMSNorm: h = u / sqrt(mean(u^2) + eps) * w)
//   x_t = sum_s mix[s, t] x_s + out[t] y           (all t from the OLD x_s)
//
// `streams_step` does the write-back of one sublayer's output y and the read for the next
// sublayer in one pass over the streams: one block a token row, the row's streams in
// registers, u in shared memory between the sum of squares and the scaling. Either half may
// be left out (no y: the first sublayer of a model; no read: the last write-back), and
// without a norm weight the plain sum u comes out (the sum of the streams before the final
// norm, with in = ones). Everything is fp32; the result is rounded once where it is stored.
// The order of all sums depends on the sizes only, never on which rows share a launch.
//
// `token_shift` blends a row with the row of the token before it in the same sequence,
//   out = h + (h_prev - h) * shift,
// taking h_prev of a sequence's first token of this step from the sequence's state, where it
// then leaves the sequence's last h of this step.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

template <int S, typename W, typename Out>
__global__ void __launch_bounds__(kThreads)
streams_step_kernel(float* __restrict__ xs, long long stream_stride, int streams, int width,
                    const float* __restrict__ y, const W* __restrict__ mix,
                    const W* __restrict__ out_w, int reduce, const W* __restrict__ in_w,
                    const W* __restrict__ norm_w, float eps, Out* __restrict__ out,
                    float* __restrict__ shift_state, const W* __restrict__ shift_w,
                    const int32_t* __restrict__ token_seq, const int32_t* __restrict__ slots,
                    int keep_state) {
  extern __shared__ float u_row[];                 // [width]
  __shared__ float scratch[33];
  __shared__ float c_mix[S * S], c_out[S], c_in[S];
  let_next_kernel_start();
  for (int i = threadIdx.x; i < S * S; i += kThreads) {
    const int from = i / S, to = i % S;
    c_mix[i] = (from < streams && to < streams)
                   ? (mix ? widen(mix[from * streams + to]) : (from == to ? 1.f : 0.f))
                   : 0.f;
  }
  for (int i = threadIdx.x; i < S; i += kThreads) {
    c_out[i] = i < streams ? (out_w ? widen(out_w[i]) : 1.f) : 0.f;
    c_in[i] = i < streams ? (in_w ? widen(in_w[i]) : 1.f) : 0.f;
  }
  wait_for_previous_kernel();
  __syncthreads();
  const long long row = blockIdx.x;
  float* x = xs + row * width;
  float sq = 0.f;
  for (int c = threadIdx.x; c < width; c += kThreads) {
    float v[S];
#pragma unroll
    for (int s = 0; s < S; ++s) v[s] = s < streams ? x[s * stream_stride + c] : 0.f;
    if (y) {
      const float yv = y[row * width + c];
      float n[S];
#pragma unroll
      for (int t = 0; t < S; ++t) {
        float acc = 0.f;
#pragma unroll
        for (int s = 0; s < S; ++s) acc = fmaf(c_mix[s * S + t], v[s], acc);
        n[t] = fmaf(c_out[t], yv, acc);
      }
#pragma unroll
      for (int s = 0; s < S; ++s) {
        v[s] = n[s];
        if (s < streams) x[s * stream_stride + c] = n[s];
      }
    }
    if (reduce) {
      float u = 0.f;
#pragma unroll
      for (int s = 0; s < S; ++s) u = fmaf(c_in[s], v[s], u);
      u_row[c] = u;
      sq = fmaf(u, u, sq);
    }
  }
  if (!reduce) return;
  float r = 1.f;
  if (norm_w) {
    const float total = block_sum(sq, scratch);
    r = 1.f / sqrtf(total / (float)width + eps);
  }
  Out* o = out + row * width;
  // With `shift_state` every row is the one token its sequence brings in this step: the blend
  // with the token before (`token_shift` below) happens here, on the normed row.
  float* kept = shift_state ? shift_state + (long long)slots[token_seq[row]] * width : nullptr;
  // (each thread reads back the columns it wrote itself)
  for (int c = threadIdx.x; c < width; c += kThreads) {
    const float cur = norm_w ? u_row[c] * r * widen(norm_w[c]) : u_row[c];
    if (kept) {
      const float prev = kept[c];
      if (keep_state) kept[c] = cur;
      o[c] = narrow<Out>(fmaf(prev - cur, widen(shift_w[c]), cur));
    } else {
      o[c] = narrow<Out>(cur);
    }
  }
}

template <typename W, typename Out>
__global__ void token_shift_kernel(const float* __restrict__ h, float* __restrict__ state,
                                   const W* __restrict__ shift,
                                   const int32_t* __restrict__ token_seq,
                                   const int32_t* __restrict__ cu_seqlens,
                                   const int32_t* __restrict__ slots, Out* __restrict__ out,
                                   int width, long long count, int keep_state) {
  let_next_kernel_start();
  wait_for_previous_kernel();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / width;
    const int c = static_cast<int>(i - t * width);
    const int seq = token_seq[t];
    const float cur = h[i];
    float prev;
    if (t == cu_seqlens[seq]) {
      // only this thread touches the sequence's state at column c: it reads the old value
      // and then leaves the value of the sequence's last row of this step
      float* kept = state + (long long)slots[seq] * width + c;
      prev = *kept;
      if (keep_state) *kept = h[(long long)(cu_seqlens[seq + 1] - 1) * width + c];
    } else {
      prev = h[i - width];
    }
    out[i] = narrow<Out>(fmaf(prev - cur, widen(shift[c]), cur));
  }
}

__global__ void streams_spread_kernel(float* __restrict__ xs, long long stream_stride,
                                      int streams, long long count) {
  let_next_kernel_start();
  wait_for_previous_kernel();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x) {
    const float v = xs[i];
    for (int s = 1; s < streams; ++s) xs[s * stream_stride + i] = v;
  }
}

template <int S, typename W>
int launch_step(float* xs, long long stride, int streams, int tokens, int width, const float* y,
                const void* mix, const void* out_w, int reduce, const void* in_w,
                const void* norm_w, float eps, void* out, int out_dtype, float* shift_state,
                const void* shift_w, const int32_t* token_seq, const int32_t* slots,
                int keep_state, cudaStream_t stream) {
  const size_t smem = reduce ? (size_t)width * sizeof(float) : 0;
  if (smem > 200 * 1024) return cudaErrorInvalidValue;
  auto go = [&](auto kernel, auto* o) {
    if (smem > 48 * 1024) {
      const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 (int)smem);
      if (e != cudaSuccess) return (int)e;
    }
    return launch_overlapped(kernel, dim3(tokens), dim3(kThreads), smem, stream, 1, xs, stride,
                             streams, width, y, (const W*)mix, (const W*)out_w, reduce,
                             (const W*)in_w, (const W*)norm_w, eps, o, shift_state,
                             (const W*)shift_w, token_seq, slots, keep_state);
  };
  if (out_dtype == SAKV_F32) return go(streams_step_kernel<S, W, float>, (float*)out);
  if (out_dtype == SAKV_BF16) return go(streams_step_kernel<S, W, __nv_bfloat16>, (__nv_bfloat16*)out);
  return cudaErrorInvalidValue;
}

template <typename W>
int pick_step(float* xs, long long stride, int streams, int tokens, int width, const float* y,
              const void* mix, const void* out_w, int reduce, const void* in_w,
              const void* norm_w, float eps, void* out, int out_dtype, float* shift_state,
              const void* shift_w, const int32_t* token_seq, const int32_t* slots,
              int keep_state, cudaStream_t stream) {
#define SAKV_STEP(S)                                                                          \
  return launch_step<S, W>(xs, stride, streams, tokens, width, y, mix, out_w, reduce, in_w,   \
                           norm_w, eps, out, out_dtype, shift_state, shift_w, token_seq, slots, \
                           keep_state, stream)
  if (streams == 1) SAKV_STEP(1);
  if (streams == 2) SAKV_STEP(2);
  if (streams <= 4) SAKV_STEP(4);
  if (streams <= 8) SAKV_STEP(8);
  SAKV_STEP(16);
#undef SAKV_STEP
}

}  // namespace

// xs: [streams, tokens, width] fp32 with `stream_stride` elements between streams. y (or
// null): [tokens, width] fp32 to write back with `mix` [streams, streams] (from, to) and
// `out_w` [streams] (null: identity and ones). `reduce` != 0: out[tokens, width] = the
// normed weighted sum (`in_w` null: ones; `norm_w` null: no norm, out must be fp32-sized
// for its type all the same). The constants are of type `w_dtype`. `shift_state` (or null):
// fp32 [slots, width]; given only when every row is the one token that its sequence
// (`token_seq`, `slots`) brings, it blends the result with the sequence's row before, as
// `sakv_token_shift` does, and leaves the unblended result there.
SAKV_EXPORT int sakv_streams_step(float* xs, long long stream_stride, int streams, int tokens,
                                  int width, const float* y, const void* mix, const void* out_w,
                                  int reduce, const void* in_w, const void* norm_w, int w_dtype,
                                  float eps, void* out, int out_dtype, float* shift_state,
                                  const void* shift_w, const int32_t* token_seq,
                                  const int32_t* slots, int keep_state, cudaStream_t stream) {
  if (streams < 1 || streams > 16 || tokens < 0 || width <= 0 || (!y && !reduce) ||
      (reduce && !out) || (shift_state && (!reduce || !shift_w || !token_seq || !slots)))
    return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  if (w_dtype == SAKV_F32)
    return pick_step<float>(xs, stream_stride, streams, tokens, width, y, mix, out_w, reduce,
                            in_w, norm_w, eps, out, out_dtype, shift_state, shift_w, token_seq,
                            slots, keep_state, stream);
  if (w_dtype == SAKV_BF16)
    return pick_step<__nv_bfloat16>(xs, stream_stride, streams, tokens, width, y, mix, out_w,
                                    reduce, in_w, norm_w, eps, out, out_dtype, shift_state,
                                    shift_w, token_seq, slots, keep_state, stream);
  return cudaErrorInvalidValue;
}

SAKV_EXPORT int sakv_token_shift(const float* h, float* state, const void* shift, int w_dtype,
                                 const int32_t* token_seq, const int32_t* cu_seqlens,
                                 const int32_t* slots, void* out, int out_dtype, int tokens,
                                 int width, int keep_state, cudaStream_t stream) {
  if (tokens < 0 || width <= 0) return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  const long long count = (long long)tokens * width;
  const dim3 grid(grid_for(count, 256)), block(256);
#define SAKV_SHIFT(W, O)                                                                        \
  return launch_overlapped(token_shift_kernel<W, O>, grid, block, 0, stream, 1, h, state,       \
                           (const W*)shift, token_seq, cu_seqlens, slots, (O*)out, width, count, \
                           keep_state)
  if (w_dtype == SAKV_F32 && out_dtype == SAKV_F32) SAKV_SHIFT(float, float);
  if (w_dtype == SAKV_F32 && out_dtype == SAKV_BF16) SAKV_SHIFT(float, __nv_bfloat16);
  if (w_dtype == SAKV_BF16 && out_dtype == SAKV_F32) SAKV_SHIFT(__nv_bfloat16, float);
  if (w_dtype == SAKV_BF16 && out_dtype == SAKV_BF16) SAKV_SHIFT(__nv_bfloat16, __nv_bfloat16);
#undef SAKV_SHIFT
  return cudaErrorInvalidValue;
}

// xs[s] = xs[0] for every further stream s.
SAKV_EXPORT int sakv_streams_spread(float* xs, long long stream_stride, int streams,
                                    long long count, cudaStream_t stream) {
  if (streams < 1 || count < 0) return cudaErrorInvalidValue;
  if (streams == 1 || count == 0) return 0;
  return launch_overlapped(streams_spread_kernel, dim3(grid_for(count, 256)), dim3(256), 0,
                           stream, 1, xs, stream_stride, streams, count);
}
