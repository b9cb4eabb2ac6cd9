// Causal grouped-query attention for steps that bring many tokens per sequence (prompts, chunks of
// prompts), bfloat16, over the paged cache.
//
// A CTA takes 64 consecutive query tokens of one sequence and one query head; its four warps hold 16
// query rows each as tensor-core fragments and walk the sequence's pages (64 keys each) up to the
// diagonal with the online softmax (running maximum, sum and accumulator in float,
// engine/kernels/fused.py:288-312; the probabilities are rounded to bfloat16 for the second product
// as fused.py:699-701 does).  Keys and values of the step's own tokens are read from the cache like
// all others, so a chunk that continues a sequence needs nothing special: a query at absolute
// position p sees keys j <= p (engine/engine.py:781-787) and, with a window w, j > p - w.
//
// Pages are copied to shared memory with 16-byte asynchronous copies, two pages ahead of the math,
// into a layout whose 16-byte columns are XOR-swizzled by the row so that ldmatrix reads without
// bank conflicts.  Products use mma.sync.m16n8k16 (bf16 in, float accumulate).
#include "common.cuh"

#define PF_BQ 64
#define PF_WARPS 4
#define PF_THREADS (PF_WARPS * 32)

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Byte offset of 16-byte column `chunk` of `row` in a [rows][D] bfloat16 tile with swizzled columns.
template <int D> __device__ __forceinline__ int tile_offset(int row, int chunk) {
  constexpr int C = D / 8;  // 16-byte columns per row
  const int sw = C >= 8 ? (row & 7) : ((row / (8 / C)) % C);
  return row * D * 2 + ((chunk ^ sw) << 4);
}

template <int D>
__global__ void __launch_bounds__(PF_THREADS)
attention_prefill_kernel(const bf16* __restrict__ q, bf16* __restrict__ out,
                         const bf16* __restrict__ k_store, const bf16* __restrict__ v_store,
                         const int* __restrict__ block_table, int table_stride,
                         const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start,
                         const int* __restrict__ seq_q_len, const int* __restrict__ seq_kv_len,
                         const int* __restrict__ tile_seq, const int* __restrict__ tile_first,
                         int heads, int kv_heads, float scale_log2, int window) {
  constexpr int C = D / 8;
  constexpr int TILE_BYTES = SB_PAGE_TOKENS * D * 2;
  constexpr int KSTEPS = D / 16;   // k steps of Q.K^T
  constexpr int NBLK = D / 8;      // 8-wide column blocks of the output
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* q_tile = smem;                       // [64][D]
  uint8_t* k_tiles = smem + PF_BQ * D * 2;      // 2 x [64][D]
  uint8_t* v_tiles = k_tiles + 2 * TILE_BYTES;  // 2 x [64][D]

  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(q);
  const int tile = blockIdx.x, head = blockIdx.y;
  const int seq = tile_seq[tile];
  const int q_first = tile_first[tile];         // first query of this tile within the step's tokens of seq
  const int q_len = seq_q_len[seq], kv_len = seq_kv_len[seq];
  const int rows_valid = min(PF_BQ, q_len - q_first);
  const int pos0 = kv_len - q_len + q_first;    // absolute position of the tile's first query
  const int kvh = head / (heads / kv_heads);
  const int* pages = block_table + (size_t)seq_slot[seq] * table_stride;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  const int hi = pos0 + rows_valid - 1;                                   // last key any row sees
  int lo = 0;
  if (window > 0 && pos0 - window + 1 > 0) lo = pos0 - window + 1;        // first key any row sees
  const int page_lo = lo / SB_PAGE_TOKENS, page_hi = hi / SB_PAGE_TOKENS;
  const int n_tiles = page_hi - page_lo + 1;

  // ---- stage the queries (rows past the end repeat the last valid row; they are never written)
  {
    const size_t row_stride = (size_t)heads * D;
    const bf16* src = q + ((size_t)seq_q_start[seq] + q_first) * row_stride + (size_t)head * D;
    for (int idx = tid; idx < PF_BQ * C; idx += PF_THREADS) {
      const int r = idx / C, c = idx % C;
      const int rr = min(r, rows_valid - 1);
      cp_async16(q_tile + tile_offset<D>(r, c), src + (size_t)rr * row_stride + c * 8);
    }
  }
  auto load_kv = [&](int t, int buf) {
    const size_t base = page_row(pages[page_lo + t], kvh, 0, kv_heads, D);
    const bf16* ks = k_store + base;
    const bf16* vs = v_store + base;
    for (int idx = tid; idx < SB_PAGE_TOKENS * C; idx += PF_THREADS) {
      const int r = idx / C, c = idx % C;
      cp_async16(k_tiles + buf * TILE_BYTES + tile_offset<D>(r, c), ks + (size_t)idx * 8);
      cp_async16(v_tiles + buf * TILE_BYTES + tile_offset<D>(r, c), vs + (size_t)idx * 8);
    }
  };
  load_kv(0, 0);
  cp_commit();
  if (n_tiles > 1) load_kv(1, 1);
  cp_commit();
  cp_wait<1>();
  __syncthreads();

  // ---- this warp's 16 query rows as A fragments
  uint32_t qf[KSTEPS][4];
  {
    const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk)
      ldmatrix_x4(smem_u32(q_tile + tile_offset<D>(r, 2 * kk + (lane >> 4))), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
  }
  float o[NBLK][4];
#pragma unroll
  for (int n = 0; n < NBLK; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const int row_a = warp * 16 + (lane >> 2);     // this thread's rows: row_a and row_a + 8
  const int pos_a = pos0 + row_a, pos_b = pos_a + 8;

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t & 1;
    const uint8_t* kt = k_tiles + buf * TILE_BYTES;
    const uint8_t* vt = v_tiles + buf * TILE_BYTES;
    const int j0 = (page_lo + t) * SB_PAGE_TOKENS;

    // S = Q K^T for 64 keys: 8 blocks of 8 keys
    float s[8][4];
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
      for (int nb = 0; nb < 8; nb += 2) {
        uint32_t b0, b1, b2, b3;
        const int key = nb * 8 + (lane & 7) + (lane >> 4) * 8;
        ldmatrix_x4(smem_u32(kt + tile_offset<D>(key, 2 * kk + ((lane >> 3) & 1))), b0, b1, b2, b3);
        mma_bf16(s[nb], qf[kk], b0, b1);
        mma_bf16(s[nb + 1], qf[kk], b2, b3);
      }
    }

    // scale, mask, online softmax
    const bool edge = j0 + SB_PAGE_TOKENS - 1 > pos0 || (window > 0 && j0 <= pos0 + PF_BQ - window);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[nb][e] * scale_log2;
        if (edge) {
          const int j = j0 + nb * 8 + (lane & 3) * 2 + (e & 1);
          const int p = (e & 2) ? pos_b : pos_a;
          if (j > p || (window > 0 && j <= p - window)) v = -INFINITY;
        }
        s[nb][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
    float alpha[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
      const float m_new = fmaxf(m_run[h], mx[h]);
      m_use[h] = m_new == -INFINITY ? 0.f : m_new;
      alpha[h] = exp2f(m_run[h] - m_use[h]);
      m_run[h] = m_new;
    }
    float rs[2] = {0.f, 0.f};
    uint32_t pf[4][4];   // P as A fragments: 4 k-steps of 16 keys
#pragma unroll
    for (int nb = 0; nb < 8; ++nb) {
      const float p0 = exp2f(s[nb][0] - m_use[0]), p1 = exp2f(s[nb][1] - m_use[0]);
      const float p2 = exp2f(s[nb][2] - m_use[1]), p3 = exp2f(s[nb][3] - m_use[1]);
      rs[0] += p0 + p1;
      rs[1] += p2 + p3;
      pf[nb >> 1][(nb & 1) * 2] = pack_bf16(p0, p1);
      pf[nb >> 1][(nb & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) l_run[h] = l_run[h] * alpha[h] + rs[h];
#pragma unroll
    for (int n = 0; n < NBLK; ++n) {
      o[n][0] *= alpha[0]; o[n][1] *= alpha[0];
      o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
    }

    // O += P V
#pragma unroll
    for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
      for (int n = 0; n < NBLK; n += 2) {
        uint32_t b0, b1, b2, b3;
        const int key = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        ldmatrix_x4_trans(smem_u32(vt + tile_offset<D>(key, n + (lane >> 4))), b0, b1, b2, b3);
        mma_bf16(o[n], pf[kk], b0, b1);
        mma_bf16(o[n + 1], pf[kk], b2, b3);
      }
    }

    // this buffer is free: fetch the tile after next, then make sure the next one has landed
    __syncthreads();
    if (t + 2 < n_tiles) load_kv(t + 2, buf);
    cp_commit();
    cp_wait<1>();
    __syncthreads();
  }
  cp_wait<0>();

  // ---- finish: rows sum over the quad, divide, store
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  const float inv_a = 1.f / l_run[0], inv_b = 1.f / l_run[1];
  const size_t row_stride = (size_t)heads * D;
  bf16* dst = out + ((size_t)seq_q_start[seq] + q_first) * row_stride + (size_t)head * D;
#pragma unroll
  for (int n = 0; n < NBLK; ++n) {
    const int col = n * 8 + (lane & 3) * 2;
    if (row_a < rows_valid)
      *reinterpret_cast<uint32_t*>(dst + (size_t)row_a * row_stride + col) = pack_bf16(o[n][0] * inv_a, o[n][1] * inv_a);
    if (row_a + 8 < rows_valid)
      *reinterpret_cast<uint32_t*>(dst + (size_t)(row_a + 8) * row_stride + col) = pack_bf16(o[n][2] * inv_b, o[n][3] * inv_b);
  }
}

template <int D>
static int launch(const void* q, void* out, const void* k_store, const void* v_store,
                  const int* block_table, int table_stride, const int* seq_slot, const int* seq_q_start,
                  const int* seq_q_len, const int* seq_kv_len, const int* tile_seq, const int* tile_first,
                  int n_tiles, int heads, int kv_heads, float scale, int window, cudaStream_t s) {
  const int smem = (PF_BQ + 4 * SB_PAGE_TOKENS) * D * 2;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return launch_dependent(attention_prefill_kernel<D>, dim3(n_tiles, heads), dim3(PF_THREADS), smem, s,
      (const bf16*)q, (bf16*)out, (const bf16*)k_store, (const bf16*)v_store, block_table, table_stride,
      seq_slot, seq_q_start, seq_q_len, seq_kv_len, tile_seq, tile_first, heads, kv_heads,
      scale * 1.4426950408889634f, window);
}

extern "C" {

// q, out: [tokens, heads * head_dim] bfloat16, packed by sequence.  Per sequence i: its slot, where
// its queries start in the packing, how many there are and its length once they are cached.  The
// work list names, per tile of 64 queries, its sequence and its first query within that sequence.
// head_dim must be 16, 32, 64 or 128 (returns -2 otherwise).
int sb_attention_prefill(const void* q, void* out, const void* k_store, const void* v_store,
                         const int* block_table, int table_stride, const int* seq_slot,
                         const int* seq_q_start, const int* seq_q_len, const int* seq_kv_len,
                         const int* tile_seq, const int* tile_first, int n_tiles, int heads,
                         int kv_heads, int head_dim, float scale, int window, cudaStream_t s) {
  if (n_tiles == 0) return 0;
  if (kv_heads <= 0 || heads % kv_heads) return -2;
#define ARGS q, out, k_store, v_store, block_table, table_stride, seq_slot, seq_q_start, seq_q_len, \
             seq_kv_len, tile_seq, tile_first, n_tiles, heads, kv_heads, scale, window, s
  switch (head_dim) {
    case 16: return launch<16>(ARGS);
    case 32: return launch<32>(ARGS);
    case 64: return launch<64>(ARGS);
    case 128: return launch<128>(ARGS);
    default: return -2;
  }
#undef ARGS
}

}  // extern "C"
