// Causal grouped-query attention over the paged cache, one warp per (query token, query head).
//
// This is the plain kernel: it serves the whole 32-bit path (prompts and single tokens alike) and any
// shape the faster bfloat16 kernels refuse.  A query at absolute position p of the sequence in `slot`
// sees key j of the same slot iff j <= p, and with a window w only iff j > p - w
// (engine/engine.py:781-787 for the rule that causality follows absolute positions, not the number of
// queries in the step).  Query head h reads key/value head h / (heads / kv_heads)
// (engine/kernels/fused.py:263-266).  Scores, the running maximum and sum, and the accumulator are
// float (fused.py:288-312); the result is rounded to the working type once.
#include "common.cuh"

#define SB_ROW_MAX_D 8  // head_dim <= 256

template <typename T>
__global__ void attention_rowwise_kernel(const T* __restrict__ q, T* __restrict__ out,
                                         const T* __restrict__ k_store, const T* __restrict__ v_store,
                                         const int* __restrict__ block_table, int table_stride,
                                         const int* __restrict__ tok_slot,
                                         const int* __restrict__ tok_pos, int n_tokens, int heads,
                                         int kv_heads, int head_dim, float scale, int window) {
  const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= (long long)n_tokens * heads) return;
  const int token = (int)(warp / heads);
  const int h = (int)(warp - (long long)token * heads);
  const int kvh = h / (heads / kv_heads);
  const int pos = tok_pos[token];
  const int* pages = block_table + (size_t)tok_slot[token] * table_stride;
  const T* qr = q + ((size_t)token * heads + h) * head_dim;

  float qv[SB_ROW_MAX_D], acc[SB_ROW_MAX_D];
#pragma unroll
  for (int i = 0; i < SB_ROW_MAX_D; ++i) {
    const int d = lane + 32 * i;
    qv[i] = d < head_dim ? to_f<T>(qr[d]) * scale : 0.f;
    acc[i] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  int first = 0;
  if (window > 0 && pos - window + 1 > 0) first = pos - window + 1;

  for (int j0 = first; j0 <= pos; j0 += 4) {
    float s[4];
    const T* vrow[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int j = j0 + u;
      s[u] = 0.f;
      vrow[u] = nullptr;
      if (j <= pos) {
        const int page = pages[j / SB_PAGE_TOKENS];
        const size_t off = page_row(page, kvh, j % SB_PAGE_TOKENS, kv_heads, head_dim);
        const T* kr = k_store + off;
        vrow[u] = v_store + off;
#pragma unroll
        for (int i = 0; i < SB_ROW_MAX_D; ++i) {
          const int d = lane + 32 * i;
          if (d < head_dim) s[u] += qv[i] * to_f<T>(kr[d]);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) s[u] = warp_sum(s[u]);
    float m_new = m;
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (j0 + u <= pos) m_new = fmaxf(m_new, s[u]);
    const float alpha = expf(m - m_new);
    l *= alpha;
#pragma unroll
    for (int i = 0; i < SB_ROW_MAX_D; ++i) acc[i] *= alpha;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (j0 + u <= pos) {
        const float p = expf(s[u] - m_new);
        l += p;
#pragma unroll
        for (int i = 0; i < SB_ROW_MAX_D; ++i) {
          const int d = lane + 32 * i;
          if (d < head_dim) acc[i] += p * to_f<T>(vrow[u][d]);
        }
      }
    }
    m = m_new;
  }
  T* orow = out + ((size_t)token * heads + h) * head_dim;
  const float inv = 1.f / l;
#pragma unroll
  for (int i = 0; i < SB_ROW_MAX_D; ++i) {
    const int d = lane + 32 * i;
    if (d < head_dim) orow[d] = from_f<T>(acc[i] * inv);
  }
}

extern "C" {

// q, out: [n_tokens, heads * head_dim].  window <= 0 means all keys.
int sb_attention_rowwise(int dtype, const void* q, void* out, const void* k_store, const void* v_store,
                         const int* block_table, int table_stride, const int* tok_slot,
                         const int* tok_pos, int n_tokens, int heads, int kv_heads, int head_dim,
                         float scale, int window, cudaStream_t s) {
  if (head_dim > 32 * SB_ROW_MAX_D || kv_heads <= 0 || heads % kv_heads) return -2;
  const long long warps = (long long)n_tokens * heads;
  if (warps == 0) return 0;
  const int threads = 128;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  if (dtype == 0)
    attention_rowwise_kernel<float><<<(unsigned)blocks, threads, 0, s>>>(
        (const float*)q, (float*)out, (const float*)k_store, (const float*)v_store, block_table,
        table_stride, tok_slot, tok_pos, n_tokens, heads, kv_heads, head_dim, scale, window);
  else
    attention_rowwise_kernel<bf16><<<(unsigned)blocks, threads, 0, s>>>(
        (const bf16*)q, (bf16*)out, (const bf16*)k_store, (const bf16*)v_store, block_table,
        table_stride, tok_slot, tok_pos, n_tokens, heads, kv_heads, head_dim, scale, window);
  return SB_LAUNCH_RESULT();
}

}  // extern "C"
