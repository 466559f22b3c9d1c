// Causal grouped-query attention with a logarithmic distance penalty, an optional window,
// values of a width of their own and an optional gate a head:
//
//   s_ij = (q_i . k_j) * scale - slope[h] * ln(1 + rate[h] * (i - j))
//          for the keys j with 0 <= i - j (< window where there is one)
//   out_i = (sum_j softmax(s_i)_j v_j) * sigmoid(gate_i[h])
//
// Scores, the penalty, the softmax weights and the weighted sum of the values are fp32; keys
// and values are widened from the cache's type. One warp for each (token, head) walks the
// visible keys in the order of their positions with a running maximum and sum, so a token's
// result is the same to the bit whether it came in a prompt, in a piece of one, alone or
// beside other sequences. `kv_store` puts a step's keys and values (columns of the fused
// projection's output) into the cache blocks: keys [block, kv_head, 64, dim], values
// [block, kv_head, 64, vdim].
#include "common.cuh"

namespace {

template <typename T>
__global__ void kv_store_kernel(const T* __restrict__ qkv, long long stride, int k_off, int v_off,
                                const int32_t* __restrict__ positions,
                                const int32_t* __restrict__ token_seq,
                                const int32_t* __restrict__ block_table, int max_blocks,
                                T* __restrict__ k_cache, T* __restrict__ v_cache, int kv_heads,
                                int dim, int vdim, long long count) {
  let_next_kernel_start();
  wait_for_previous_kernel();
  const int per_token = kv_heads * (dim + vdim);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < count;
       i += (long long)gridDim.x * blockDim.x) {
    const long long t = i / per_token;
    int c = static_cast<int>(i - t * per_token);
    const int pos = positions[t];
    const int block = block_table[(long long)token_seq[t] * max_blocks + pos / kCacheBlock];
    const int at = pos % kCacheBlock;
    if (c < kv_heads * dim) {
      const int g = c / dim, e = c - g * dim;
      k_cache[(((long long)block * kv_heads + g) * kCacheBlock + at) * dim + e] =
          qkv[t * stride + k_off + c];
    } else {
      c -= kv_heads * dim;
      const int g = c / vdim, e = c - g * vdim;
      v_cache[(((long long)block * kv_heads + g) * kCacheBlock + at) * vdim + e] =
          qkv[t * stride + v_off + c];
    }
  }
}

template <int PER, typename T>
__global__ void distance_attention_kernel(
    const T* __restrict__ qkv, long long stride, int gate_off, T* __restrict__ out,
    const T* __restrict__ k_cache, const T* __restrict__ v_cache,
    const int32_t* __restrict__ positions, const int32_t* __restrict__ token_seq,
    const int32_t* __restrict__ block_table, int max_blocks, int tokens, int heads, int kv_heads,
    int dim, int vdim, float scale, int window, const float* __restrict__ slope,
    const float* __restrict__ rate) {
  let_next_kernel_start();
  wait_for_previous_kernel();
  const long long warp = (blockIdx.x * (long long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (long long)tokens * heads) return;
  const int t = static_cast<int>(warp / heads);
  const int h = static_cast<int>(warp - (long long)t * heads);
  const int g = h / (heads / kv_heads);
  const int pos = positions[t];
  const int32_t* table = block_table + (long long)token_seq[t] * max_blocks;
  const float sl = slope ? slope[h] : 0.f, rt = rate ? rate[h] : 0.f;

  float qr[PER], acc[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    qr[i] = e < dim ? widen(qkv[(long long)t * stride + (long long)h * dim + e]) : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  const int first = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  for (int j = first; j <= pos; ++j) {
    const int block = table[j / kCacheBlock];
    const long long at = ((long long)block * kv_heads + g) * kCacheBlock + j % kCacheBlock;
    const T* kp = k_cache + at * dim;
    const T* vp = v_cache + at * vdim;
    float part = 0.f;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + 32 * i;
      if (e < dim) part = fmaf(qr[i], widen(kp[e]), part);
    }
    float s = warp_sum(part) * scale;
    if (slope) s -= sl * log1pf(rt * (float)(pos - j));
    const float m_new = fmaxf(m, s);
    const float corr = expf(m - m_new);
    const float p = expf(s - m_new);
    l = fmaf(l, corr, p);
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int e = lane + 32 * i;
      if (e < vdim) acc[i] = fmaf(acc[i], corr, p * widen(vp[e]));
    }
    m = m_new;
  }
  float gate = 1.f;
  if (gate_off >= 0) {
    const float z = widen(qkv[(long long)t * stride + gate_off + h]);
    gate = 1.f / (1.f + expf(-z));
  }
  const float inv = gate / l;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int e = lane + 32 * i;
    if (e < vdim) out[((long long)t * heads + h) * vdim + e] = narrow<T>(acc[i] * inv);
  }
}

template <typename T>
int launch_attention(const void* qkv, long long stride, int gate_off, void* out,
                     const void* k_cache, const void* v_cache, const int32_t* positions,
                     const int32_t* token_seq, const int32_t* block_table, int max_blocks,
                     int tokens, int heads, int kv_heads, int dim, int vdim, float scale,
                     int window, const float* slope, const float* rate, cudaStream_t stream) {
  const int threads = 128;
  const long long blocks = ((long long)tokens * heads * 32 + threads - 1) / threads;
  if (blocks > 0x7fffffffLL) return cudaErrorInvalidValue;
  const int widest = dim > vdim ? dim : vdim;
#define SAKV_ATT(PER)                                                                            \
  return launch_overlapped(distance_attention_kernel<PER, T>, dim3((unsigned)blocks),            \
                           dim3(threads), 0, stream, 1, (const T*)qkv, stride, gate_off, (T*)out, \
                           (const T*)k_cache, (const T*)v_cache, positions, token_seq,           \
                           block_table, max_blocks, tokens, heads, kv_heads, dim, vdim, scale,   \
                           window, slope, rate)
  if (widest <= 32) SAKV_ATT(1);
  if (widest <= 64) SAKV_ATT(2);
  if (widest <= 128) SAKV_ATT(4);
  if (widest <= 256) SAKV_ATT(8);
  SAKV_ATT(16);
#undef SAKV_ATT
}

}  // namespace

SAKV_EXPORT int sakv_kv_store(const void* qkv, int dtype, long long stride, int k_off, int v_off,
                              const int32_t* positions, const int32_t* token_seq,
                              const int32_t* block_table, int max_blocks, void* k_cache,
                              void* v_cache, int tokens, int kv_heads, int dim, int vdim,
                              cudaStream_t stream) {
  if (tokens < 0 || kv_heads <= 0 || dim <= 0 || vdim <= 0 || max_blocks <= 0)
    return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  const long long count = (long long)tokens * kv_heads * (dim + vdim);
  const dim3 grid(grid_for(count, 256)), block(256);
  if (dtype == SAKV_F32)
    return launch_overlapped(kv_store_kernel<float>, grid, block, 0, stream, 1, (const float*)qkv,
                             stride, k_off, v_off, positions, token_seq, block_table, max_blocks,
                             (float*)k_cache, (float*)v_cache, kv_heads, dim, vdim, count);
  if (dtype == SAKV_BF16)
    return launch_overlapped(kv_store_kernel<__nv_bfloat16>, grid, block, 0, stream, 1,
                             (const __nv_bfloat16*)qkv, stride, k_off, v_off, positions, token_seq,
                             block_table, max_blocks, (__nv_bfloat16*)k_cache,
                             (__nv_bfloat16*)v_cache, kv_heads, dim, vdim, count);
  return cudaErrorInvalidValue;
}

// qkv: [tokens, stride] with the queries in its first heads * dim columns and, if gate_off
// >= 0, the gates' pre-activations in columns gate_off .. gate_off + heads - 1. slope, rate:
// fp32 [heads] (null: no penalty). window 0: every earlier key. out: [tokens, heads * vdim].
SAKV_EXPORT int sakv_distance_attention(const void* qkv, int dtype, long long stride, int gate_off,
                                        void* out, const void* k_cache, const void* v_cache,
                                        const int32_t* positions, const int32_t* token_seq,
                                        const int32_t* block_table, int max_blocks, int tokens,
                                        int heads, int kv_heads, int dim, int vdim, float scale,
                                        int window, const float* slope, const float* rate,
                                        cudaStream_t stream) {
  if (tokens < 0 || heads <= 0 || kv_heads <= 0 || heads % kv_heads || dim <= 0 || vdim <= 0 ||
      dim > 512 || vdim > 512 || max_blocks <= 0 || window < 0)
    return cudaErrorInvalidValue;
  if (tokens == 0) return 0;
  if (dtype == SAKV_F32)
    return launch_attention<float>(qkv, stride, gate_off, out, k_cache, v_cache, positions,
                                   token_seq, block_table, max_blocks, tokens, heads, kv_heads,
                                   dim, vdim, scale, window, slope, rate, stream);
  if (dtype == SAKV_BF16)
    return launch_attention<__nv_bfloat16>(qkv, stride, gate_off, out, k_cache, v_cache,
                                           positions, token_seq, block_table, max_blocks, tokens,
                                           heads, kv_heads, dim, vdim, scale, window, slope, rate,
                                           stream);
  return cudaErrorInvalidValue;
}
