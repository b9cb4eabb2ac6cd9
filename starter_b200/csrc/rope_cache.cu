// Per-head q/k RMSNorm, rotary positions and the write of keys and values into the paged cache, in
// one pass over the fused projection output.  One warp per (token, head) row of head_dim values.
//
// Formulas (engine/engine.py:699-718, engine/kernels/fused.py:161-219 and 553-617): the head row is
// normed with the gain shared by all heads (normalised value rounded to the working type, then times
// the gain), then rotated half-split: out[j] = n[j]*cos[j] - n[j+half]*sin[j], out[j+half] =
// n[j+half]*cos[j] + n[j]*sin[j], each product and the sum rounded to the working type, cos and sin
// rounded to the working type first.  Values are copied unchanged.  The cache position of a token is
// its absolute position in its sequence: page block_table[slot][pos / 64], offset pos % 64.
#include "common.cuh"

#define SB_MAX_PAIRS 4  // head_dim <= 256

template <typename T, typename W>
__global__ void qk_norm_rope_store_kernel(
    const T* __restrict__ qkv, T* __restrict__ q_out, const W* __restrict__ q_gain,
    const W* __restrict__ k_gain, const float* __restrict__ cos_table,
    const float* __restrict__ sin_table, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_slot, const int* __restrict__ block_table, int table_stride,
    T* __restrict__ k_store, T* __restrict__ v_store, int n_tokens, int heads, int kv_heads,
    int head_dim, float eps, int heads_per_token, int row_stride) {
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(qkv);
  SB_BEHIND_WAIT(tok_pos);
  SB_BEHIND_WAIT(tok_slot);
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= n_tokens * heads_per_token) return;
  const int token = warp / heads_per_token;
  const int h = warp - token * heads_per_token;
  const int half = head_dim >> 1;
  const T* src = qkv + (size_t)token * row_stride + (size_t)h * head_dim;
  const int pos = tok_pos[token];

  T* dst;
  const bool is_q = h < heads;
  const bool is_v = h >= heads + kv_heads;
  if (is_q) {
    dst = q_out + ((size_t)token * heads + h) * head_dim;
  } else {
    const int kvh = is_v ? h - heads - kv_heads : h - heads;
    const int page = block_table[(size_t)tok_slot[token] * table_stride + pos / SB_PAGE_TOKENS];
    T* store = is_v ? v_store : k_store;
    dst = store + page_row(page, kvh, pos % SB_PAGE_TOKENS, kv_heads, head_dim);
  }

  if (is_v) {
    for (int d = lane; d < head_dim; d += 32) dst[d] = src[d];
    return;
  }

  float lo[SB_MAX_PAIRS], hi[SB_MAX_PAIRS];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < SB_MAX_PAIRS; ++i) {
    const int j = lane + 32 * i;
    lo[i] = hi[i] = 0.f;
    if (j < half) {
      lo[i] = to_f<T>(src[j]);
      hi[i] = to_f<T>(src[j + half]);
      ss += lo[i] * lo[i] + hi[i] * hi[i];
    }
  }
  const W* gain = is_q ? q_gain : k_gain;
  if (gain) {
    ss = warp_sum(ss);
    const float inv = rsqrtf(ss / (float)head_dim + eps);
#pragma unroll
    for (int i = 0; i < SB_MAX_PAIRS; ++i) {
      const int j = lane + 32 * i;
      if (j < half) {
        lo[i] = rnd<T>(rnd<T>(lo[i] * inv) * to_f<W>(gain[j]));
        hi[i] = rnd<T>(rnd<T>(hi[i] * inv) * to_f<W>(gain[j + half]));
      }
    }
  }
#pragma unroll
  for (int i = 0; i < SB_MAX_PAIRS; ++i) {
    const int j = lane + 32 * i;
    if (j < half) {
      float out_lo = lo[i], out_hi = hi[i];
      if (cos_table) {
        const float c = rnd<T>(cos_table[(size_t)pos * half + j]);
        const float s = rnd<T>(sin_table[(size_t)pos * half + j]);
        out_lo = rnd<T>(rnd<T>(lo[i] * c) + rnd<T>(-hi[i] * s));
        out_hi = rnd<T>(rnd<T>(hi[i] * c) + rnd<T>(lo[i] * s));
      }
      dst[j] = from_f<T>(out_lo);
      dst[j + half] = from_f<T>(out_hi);
    }
  }
}

// Eight consecutive gains as floats, with 16-byte loads where the pointer allows it.
__device__ __forceinline__ void load8(const float* p, float* out) {
  if (((uintptr_t)p & 15) == 0) {
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w; out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = p[i];
  }
}
__device__ __forceinline__ void load8(const bf16* p, float* out) {
  if (((uintptr_t)p & 15) == 0) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      out[2 * i] = __uint_as_float(w[i] << 16);
      out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = __bfloat162float(p[i]);
  }
}

// The same for bfloat16 with 16-byte accesses: L = head_dim / 16 lanes share a head row, each holding
// 8 elements of the low half and the 8 they pair with in the high half; a warp takes 32 / L rows.
template <typename W, int L>
__global__ void qk_norm_rope_store_vec_kernel(
    const bf16* __restrict__ qkv, bf16* __restrict__ q_out, const W* __restrict__ q_gain,
    const W* __restrict__ k_gain, const float* __restrict__ cos_table,
    const float* __restrict__ sin_table, const int* __restrict__ tok_pos,
    const int* __restrict__ tok_slot, const int* __restrict__ block_table, int table_stride,
    bf16* __restrict__ k_store, bf16* __restrict__ v_store, long long n_rows, int heads, int kv_heads,
    float eps, int heads_per_token, int row_stride) {
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(qkv);
  SB_BEHIND_WAIT(tok_pos);
  SB_BEHIND_WAIT(tok_slot);
  constexpr int HALF = L * 8, D = 2 * HALF;
  // grid (tokens, blocks of heads): no index needs a division
  const int token = blockIdx.x;
  const int head_here = (blockIdx.y * blockDim.x + threadIdx.x) / L;
  const int part = threadIdx.x % L;
  const bool live = head_here < heads_per_token;
  const int h = live ? head_here : 0;
  const bf16* src = qkv + (size_t)token * row_stride + (size_t)h * D + part * 8;
  const int pos = tok_pos[token];
  const bool is_q = h < heads;
  const bool is_v = h >= heads + kv_heads;
  bf16* dst;
  if (is_q) {
    dst = q_out + ((size_t)token * heads + h) * D;
  } else {
    const int kvh = is_v ? h - heads - kv_heads : h - heads;
    const int page = block_table[(size_t)tok_slot[token] * table_stride + pos / SB_PAGE_TOKENS];
    dst = (is_v ? v_store : k_store) + page_row(page, kvh, pos % SB_PAGE_TOKENS, kv_heads, D);
  }
  dst += part * 8;
  uint4 raw_lo = *reinterpret_cast<const uint4*>(src);
  uint4 raw_hi = *reinterpret_cast<const uint4*>(src + HALF);
  if (is_v) {
    if (live) {
      *reinterpret_cast<uint4*>(dst) = raw_lo;
      *reinterpret_cast<uint4*>(dst + HALF) = raw_hi;
    }
    // the shuffles below need every lane of a row's group; value rows fall in whole groups
  }
  float lo[8], hi[8];
  {
    const uint32_t wl[4] = {raw_lo.x, raw_lo.y, raw_lo.z, raw_lo.w}, wh[4] = {raw_hi.x, raw_hi.y, raw_hi.z, raw_hi.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      lo[2 * i] = __uint_as_float(wl[i] << 16); lo[2 * i + 1] = __uint_as_float(wl[i] & 0xffff0000u);
      hi[2 * i] = __uint_as_float(wh[i] << 16); hi[2 * i + 1] = __uint_as_float(wh[i] & 0xffff0000u);
    }
  }
  const W* gain = is_q ? q_gain : k_gain;
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) ss += lo[i] * lo[i] + hi[i] * hi[i];
#pragma unroll
  for (int o = L / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if (is_v || !live) return;
  if (gain) {
    const float inv = rsqrtf(ss / (float)D + eps);
    float g_lo[8], g_hi[8];
    load8(gain + part * 8, g_lo);
    load8(gain + HALF + part * 8, g_hi);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float a = lo[i] * inv, b = hi[i] * inv;
      rnd2<bf16>(a, b);
      a *= g_lo[i];
      b *= g_hi[i];
      rnd2<bf16>(a, b);
      lo[i] = a;
      hi[i] = b;
    }
  }
  if (cos_table) {
    // rows of the tables are HALF = 8 L floats: 32-byte aligned pieces
    const float4* cp4 = reinterpret_cast<const float4*>(cos_table + (size_t)pos * HALF + part * 8);
    const float4* sp4 = reinterpret_cast<const float4*>(sin_table + (size_t)pos * HALF + part * 8);
    const float4 c0 = cp4[0], c1 = cp4[1], s0 = sp4[0], s1 = sp4[1];
    const float cp[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sp[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      float c = cp[i], sn = sp[i];
      rnd2<bf16>(c, sn);
      float a0 = lo[i] * c, a1 = -hi[i] * sn, b0 = hi[i] * c, b1 = lo[i] * sn;
      rnd2<bf16>(a0, a1);
      rnd2<bf16>(b0, b1);
      float a = a0 + a1, b = b0 + b1;
      rnd2<bf16>(a, b);
      lo[i] = a;
      hi[i] = b;
    }
  }
  uint4 out_lo, out_hi;
  {
    uint32_t wl[4], wh[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {             // every value is a bfloat16 already (or came in as one)
      wl[i] = pack_exact_bf16(lo[2 * i], lo[2 * i + 1]);
      wh[i] = pack_exact_bf16(hi[2 * i], hi[2 * i + 1]);
    }
    out_lo = make_uint4(wl[0], wl[1], wl[2], wl[3]);
    out_hi = make_uint4(wh[0], wh[1], wh[2], wh[3]);
  }
  *reinterpret_cast<uint4*>(dst) = out_lo;
  *reinterpret_cast<uint4*>(dst + HALF) = out_hi;
}

template <typename W, int L>
static int launch_vec(const void* qkv, void* q_out, const void* q_gain, const void* k_gain,
                      const float* cos_table, const float* sin_table, const int* tok_pos,
                      const int* tok_slot, const int* block_table, int table_stride, void* k_store,
                      void* v_store, int n_tokens, int heads, int kv_heads, float eps, int write_cache,
                      int row_stride, cudaStream_t s) {
  const int per_token = write_cache ? heads + 2 * kv_heads : heads;
  const long long rows = (long long)n_tokens * per_token;
  if (rows == 0) return 0;
  const int threads = 128;
  const int head_blocks = (per_token * L + threads - 1) / threads;
  return launch_dependent(qk_norm_rope_store_vec_kernel<W, L>, dim3((unsigned)n_tokens, (unsigned)head_blocks), dim3(threads), 0, s,
      (const bf16*)qkv, (bf16*)q_out, (const W*)q_gain, (const W*)k_gain, cos_table, sin_table, tok_pos,
      tok_slot, block_table, table_stride, (bf16*)k_store, (bf16*)v_store, rows, heads, kv_heads, eps,
      per_token, row_stride);
}

template <typename W>
static int launch_vec_by_dim(int head_dim, const void* qkv, void* q_out, const void* q_gain,
                             const void* k_gain, const float* cos_table, const float* sin_table,
                             const int* tok_pos, const int* tok_slot, const int* block_table,
                             int table_stride, void* k_store, void* v_store, int n_tokens, int heads,
                             int kv_heads, float eps, int write_cache, int row_stride, cudaStream_t s) {
#define VARGS qkv, q_out, q_gain, k_gain, cos_table, sin_table, tok_pos, tok_slot, block_table, \
              table_stride, k_store, v_store, n_tokens, heads, kv_heads, eps, write_cache, row_stride, s
  switch (head_dim) {
    case 16: return launch_vec<W, 1>(VARGS);
    case 32: return launch_vec<W, 2>(VARGS);
    case 64: return launch_vec<W, 4>(VARGS);
    case 128: return launch_vec<W, 8>(VARGS);
    case 256: return launch_vec<W, 16>(VARGS);
    default: return -2;
  }
#undef VARGS
}

template <typename T, typename W>
static int launch(const void* qkv, void* q_out, const void* q_gain, const void* k_gain,
                  const float* cos_table, const float* sin_table, const int* tok_pos,
                  const int* tok_slot, const int* block_table, int table_stride, void* k_store,
                  void* v_store, int n_tokens, int heads, int kv_heads, int head_dim, float eps,
                  int write_cache, int row_stride, cudaStream_t s) {
  const int per_token = write_cache ? heads + 2 * kv_heads : heads;
  const long long warps = (long long)n_tokens * per_token;
  if (warps == 0) return 0;
  const int threads = 128;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  return launch_dependent(qk_norm_rope_store_kernel<T, W>, dim3((unsigned)blocks), dim3(threads), 0, s,
      (const T*)qkv, (T*)q_out, (const W*)q_gain, (const W*)k_gain, cos_table, sin_table, tok_pos,
      tok_slot, block_table, table_stride, (T*)k_store, (T*)v_store, n_tokens, heads, kv_heads,
      head_dim, eps, per_token, row_stride);
}

extern "C" {

// qkv: [n_tokens, (heads + 2*kv_heads) * head_dim]; q_out: [n_tokens, heads * head_dim].
// q_gain / k_gain may be null (no per-head norm); cos_table / sin_table [positions, head_dim/2]
// float may be null (no rotation).  Rows of qkv are row_stride elements apart.  With
// write_cache == 0 only the query heads are processed, so qkv may hold the queries alone.
int sb_qk_norm_rope_store(int dtype, int gain_dtype, const void* qkv, void* q_out, const void* q_gain,
                          const void* k_gain, const float* cos_table, const float* sin_table,
                          const int* tok_pos, const int* tok_slot, const int* block_table,
                          int table_stride, void* k_store, void* v_store, int n_tokens, int heads,
                          int kv_heads, int head_dim, float eps, int write_cache, int row_stride,
                          cudaStream_t s) {
  if (head_dim > 64 * SB_MAX_PAIRS || (head_dim & 1)) return -2;
#define ARGS qkv, q_out, q_gain, k_gain, cos_table, sin_table, tok_pos, tok_slot, block_table, \
             table_stride, k_store, v_store, n_tokens, heads, kv_heads, head_dim, eps, write_cache, \
             row_stride, s
  // bfloat16 with a power-of-two head size and 16-byte aligned rows takes the 16-byte kernel
  const bool pow2 = head_dim >= 16 && head_dim <= 256 && (head_dim & (head_dim - 1)) == 0;
  const bool aligned = row_stride % 8 == 0 && (((uintptr_t)qkv | (uintptr_t)q_out | (uintptr_t)k_store |
                                                (uintptr_t)v_store | (uintptr_t)cos_table |
                                                (uintptr_t)sin_table) & 15) == 0;
  if (dtype == 1 && pow2 && aligned) {
    if (gain_dtype == 1)
      return launch_vec_by_dim<bf16>(head_dim, qkv, q_out, q_gain, k_gain, cos_table, sin_table, tok_pos,
                                     tok_slot, block_table, table_stride, k_store, v_store, n_tokens,
                                     heads, kv_heads, eps, write_cache, row_stride, s);
    if (gain_dtype == 0)
      return launch_vec_by_dim<float>(head_dim, qkv, q_out, q_gain, k_gain, cos_table, sin_table, tok_pos,
                                      tok_slot, block_table, table_stride, k_store, v_store, n_tokens,
                                      heads, kv_heads, eps, write_cache, row_stride, s);
  }
  if (dtype == 0 && gain_dtype == 0) return launch<float, float>(ARGS);
  if (dtype == 1 && gain_dtype == 1) return launch<bf16, bf16>(ARGS);
  if (dtype == 1 && gain_dtype == 0) return launch<bf16, float>(ARGS);
#undef ARGS
  return -1;
}

}  // extern "C"
