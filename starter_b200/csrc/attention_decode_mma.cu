// Single-token attention over the paged cache on tensor cores (bfloat16), split over the keys.
//
// The CUDA-core decode kernel (attention_decode.cu) spends about a hundred instructions per key and
// head group, which at large batch costs more time than reading the keys.  Here the query heads that
// share a key/value head (engine/kernels/fused.py:641-709) form the 16 rows of an mma.sync tile
// (rows past the group are zero), the keys are its columns, and a key costs a handful of
// instructions.  Grid (row, kv_head * head_chunks, split) as in the CUDA-core kernel.  Up to 8 splits
// are the blocks of one thread-block cluster and merge through distributed shared memory; more use
// the scratch buffers and the merge kernel (fused.py:729-823).
//
// FUSED: the kernel takes the q/k/v product's output instead of finished queries and does what
// rope_cache.cu does for one-token steps itself, with the same arithmetic: each block normalises and
// rotates its own query heads; a block whose split holds the newest position does the same for the
// new key, patches key and value into its shared-memory copy of the last page, and the block of the
// first head chunk also writes them into the cache for the steps to come.  That saves a launch per
// layer, which at small batch costs more than the arithmetic.
//
// A CTA walks the pages of its split.  All four warps copy a page (keys and values, 64 x head_dim
// each) into a ring of shared-memory stages with 16-byte asynchronous copies, three pages ahead,
// XOR-swizzled for ldmatrix; each warp then takes 16 of the page's 64 keys: S = Q K^T (16 x 16),
// online softmax in float (fused.py:288-312), P rounded to bfloat16 (fused.py:699-701), O += P V.
// The warps' partial results are merged through shared memory at the end.  Lengths are read from
// device memory, per row, so one captured launch serves every step (fused.py:262-271).
#include "common.cuh"

#define DM_WARPS 4
#define DM_THREADS (DM_WARPS * 32)
#define DM_STAGES 3
#define DM_ROWS 16
#define DM_TABLE_CACHE 512
#define DM_CLUSTER_MAX 8

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
__device__ __forceinline__ uint32_t cluster_addr(uint32_t addr, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(addr), "r"(rank));
  return a;
}
__device__ __forceinline__ float cluster_load(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
// A rendezvous that publishes nothing (a releasing arrive would first wait for the output's stores).
__device__ __forceinline__ void cluster_rendezvous() {
  asm volatile("barrier.cluster.arrive.relaxed;\n\tbarrier.cluster.wait;" ::: "memory");
}
template <int D> __device__ __forceinline__ int tile_offset(int row, int chunk) {
  constexpr int C = D / 8;
  const int sw = C >= 8 ? (row & 7) : ((row / (8 / C)) % C);
  return row * D * 2 + ((chunk ^ sw) << 4);
}

// CLUSTER: the splits of a row and key/value head are the blocks of one thread-block cluster
// (cluster dimension z = n_splits <= 8) and merge their results through distributed shared memory,
// in split order, instead of through the scratch buffers and the merge kernel.
struct FusedRope {
  int q_stride;                 // elements between rows of the q/k/v product's output
  int has_kv;                   // the output holds keys and values and this layer writes its cache
  int gain_f32;                 // the head norms' gains are float (else bfloat16)
  float eps;
  const void* q_gain;           // may be null: no head norm
  const void* k_gain;
  const float* cos_table;       // [positions, D / 2]; may be null: no rotation
  const float* sin_table;
  int early;                    // lengths and older cache pages may be read before the wait (see below)
};

template <int D, bool CLUSTER, bool FUSED>
__global__ void __launch_bounds__(DM_THREADS)
attention_decode_mma_kernel(const bf16* __restrict__ q, bf16* __restrict__ out,
                            const bf16* __restrict__ k_store, const bf16* __restrict__ v_store,
                            const int* __restrict__ block_table, int table_stride,
                            const int* __restrict__ row_slot, const int* __restrict__ row_kv_len,
                            int heads, int kv_heads, float scale_log2, int window, int n_splits,
                            float* __restrict__ part_acc, float* __restrict__ part_ml, const FusedRope fr) {
  constexpr int C = D / 8;
  constexpr int PAGE_BYTES = SB_PAGE_TOKENS * D * 2;
  constexpr int STAGE_BYTES = 2 * PAGE_BYTES;
  constexpr int KSTEPS = D / 16;
  constexpr int NBLK = D / 8;
  extern __shared__ __align__(128) uint8_t smem[];
  uint8_t* q_tile = smem;                          // [16][D] bfloat16
  uint8_t* ring = smem + DM_ROWS * D * 2;          // DM_STAGES x (keys, values)
  __shared__ float sh_m[DM_WARPS][DM_ROWS], sh_l[DM_WARPS][DM_ROWS];
  __shared__ float cl_m[DM_ROWS], cl_l[DM_ROWS];   // this block's merged maximum and sum (CLUSTER)
  __shared__ __align__(16) bf16 new_kv[2][D];      // the step's own key and value (FUSED)
  __shared__ int sh_pages[DM_TABLE_CACHE];         // the row's page table

  pdl_trigger();
  const int groups = heads / kv_heads;
  const int chunks = (groups + DM_ROWS - 1) / DM_ROWS;
  const int row = blockIdx.x;
  const int kvh = blockIdx.y / chunks;
  const int g0 = (blockIdx.y % chunks) * DM_ROWS;
  const int gc = min(DM_ROWS, groups - g0);
  const int split = blockIdx.z;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // Before the dependent-launch wait only what the host wrote before the step's first kernel (the
  // row's slot and its page table, copied into shared memory) and weights (the gains) are read.  The
  // row's length is not among them: the step before advances it, and its last kernel may still run
  // when this one starts.  After the wait the order is: the length; then, together, the first pages'
  // copies (page numbers are at hand), the rotation table's row and this thread's share of the
  // q/k/v product's row; then the arithmetic on what has arrived meanwhile.
  const int slot = row_slot[row];
  const int* pages = block_table + (size_t)slot * table_stride;
  if (table_stride <= DM_TABLE_CACHE) {
    for (int i = tid; i < table_stride; i += DM_THREADS) sh_pages[i] = pages[i];
    pages = sh_pages;
  }
  constexpr int L = D / 16, HALF = D / 2, PER_PASS = DM_THREADS / L;
  const int part = tid % L;
  const bf16* in_row = FUSED ? q + (size_t)row * fr.q_stride : nullptr;   // laundered after the wait, see there
  // the item of a pass: 0..15 are the tile's query heads, 16 is the new key (FUSED)
  auto item_source = [&](int item) {
    return in_row + (size_t)(item == DM_ROWS ? heads + kvh : kvh * groups + g0 + item) * D + part * 8;
  };
  auto item_loadable = [&](int item) { return item == DM_ROWS ? fr.has_kv != 0 : item < gc; };
  float gq_lo[8], gq_hi[8];
  if (FUSED) {
    const void* gain = tid / L == DM_ROWS ? fr.k_gain : fr.q_gain;
    if (gain) {
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        gq_lo[i] = fr.gain_f32 ? ((const float*)gain)[part * 8 + i] : __bfloat162float(((const bf16*)gain)[part * 8 + i]);
        gq_hi[i] = fr.gain_f32 ? ((const float*)gain)[HALF + part * 8 + i] : __bfloat162float(((const bf16*)gain)[HALF + part * 8 + i]);
      }
    }
  }
  // EARLY (fr.early): the caller vouches that the step's first kernel was an ordinary launch, so
  // whatever earlier steps wrote (the row's length, every cached key and value but this step's own,
  // which this very kernel makes) was complete before any kernel of this step started, and that no
  // other kernel of this step writes them.  Then the length, the page numbers, the rotation table's
  // row and the first pages' copies do not wait for the q/k/v product: they are under way while it
  // still runs.  What the product wrote is read behind the wait, through laundered pointers
  // (SB_BEHIND_WAIT: without them the compiler moved the q/k/v row's loads up among the copies).
  const bool early = FUSED && fr.early;
  if (!early) {
    pdl_wait();
    SB_BEHIND_WAIT(row_kv_len);                        // the step before's sampling kernel advances it
  }
  __syncthreads();                                     // the page table is in shared memory
  const int kv_len = row_kv_len[row];
  int first = 0;
  if (window > 0 && kv_len - window > 0) first = kv_len - window;
  const int first_page = first / SB_PAGE_TOKENS;
  const int end_page = (kv_len + SB_PAGE_TOKENS - 1) / SB_PAGE_TOKENS;
  const int per_split = (end_page - first_page + n_splits - 1) / n_splits;
  const int p_begin = first_page + split * per_split;
  const int p_end = min(p_begin + per_split, end_page);
  const int n_pages = max(p_end - p_begin, 0);
  // patch: this block's pages end with the newest position, whose key and value it makes itself
  const bool patch = FUSED && fr.has_kv && n_pages > 0 && p_end == end_page;
  const int pos = kv_len - 1;

  int first_pages[DM_STAGES - 1];
#pragma unroll
  for (int i = 0; i < DM_STAGES - 1; ++i) first_pages[i] = i < n_pages ? pages[p_begin + i] : 0;
  float cs[8], sn[8];
  if (FUSED && fr.cos_table) {
    const float* cp = fr.cos_table + (size_t)pos * HALF + part * 8;
    const float* sp = fr.sin_table + (size_t)pos * HALF + part * 8;
#pragma unroll
    for (int i = 0; i < 8; ++i) { cs[i] = cp[i]; sn[i] = sp[i]; }
  }
  auto copy_page = [&](int i, int page) {
    if (i < n_pages) {
      const size_t base = page_row(page, kvh, 0, kv_heads, D);
      uint8_t* dst = ring + (size_t)(i % DM_STAGES) * STAGE_BYTES;
      for (int idx = tid; idx < SB_PAGE_TOKENS * C; idx += DM_THREADS) {
        const int r = idx / C, c = idx % C;
        cp_async16(dst + tile_offset<D>(r, c), k_store + base + (size_t)idx * 8);
        cp_async16(dst + PAGE_BYTES + tile_offset<D>(r, c), v_store + base + (size_t)idx * 8);
      }
    }
    cp_commit();
  };
  auto load_page = [&](int i) { copy_page(i, i < n_pages ? pages[p_begin + i] : 0); };
#pragma unroll
  for (int i = 0; i < DM_STAGES - 1; ++i) copy_page(i, first_pages[i]);
  if (early) pdl_wait();                               // from here on: what the q/k/v product wrote
  SB_BEHIND_WAIT(in_row);
  SB_BEHIND_WAIT(q);
  // this thread's share of the product's row for the first pass
  uint4 raw_lo0 = make_uint4(0, 0, 0, 0), raw_hi0 = make_uint4(0, 0, 0, 0);
  if (FUSED && item_loadable(tid / L)) {
    raw_lo0 = *reinterpret_cast<const uint4*>(item_source(tid / L));
    raw_hi0 = *reinterpret_cast<const uint4*>(item_source(tid / L) + HALF);
  }

  // ---- the group's queries: row r of the tile is head g0 + r; rows past the group are zero
  if (!FUSED) {
    for (int idx = tid; idx < DM_ROWS * C; idx += DM_THREADS) {
      const int r = idx / C, c = idx % C;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (r < gc) v = *reinterpret_cast<const uint4*>(q + ((size_t)row * heads + (size_t)kvh * groups + g0 + r) * D + c * 8);
      *reinterpret_cast<uint4*>(q_tile + tile_offset<D>(r, c)) = v;
    }
  } else {
    // Head norm and rotation as in rope_cache.cu's 16-byte kernel, sum order included: L lanes share
    // a head, each with 8 elements of the low half and the 8 they pair with in the high half.
#pragma unroll 1
    for (int base = 0; base < DM_ROWS + 1; base += PER_PASS) {
      const int item = base + tid / L;
      const bool is_k = item == DM_ROWS;
      const bool valid = is_k ? patch : (item < gc);
      uint4 raw_lo = raw_lo0, raw_hi = raw_hi0;
      if (base > 0) {                                  // the first pass's loads are long under way
        raw_lo = raw_hi = make_uint4(0, 0, 0, 0);
        if (valid && item <= DM_ROWS) {
          raw_lo = *reinterpret_cast<const uint4*>(item_source(item));
          raw_hi = *reinterpret_cast<const uint4*>(item_source(item) + HALF);
        }
        const void* gain = is_k ? fr.k_gain : fr.q_gain;
        if (gain) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            gq_lo[i] = fr.gain_f32 ? ((const float*)gain)[part * 8 + i] : __bfloat162float(((const bf16*)gain)[part * 8 + i]);
            gq_hi[i] = fr.gain_f32 ? ((const float*)gain)[HALF + part * 8 + i] : __bfloat162float(((const bf16*)gain)[HALF + part * 8 + i]);
          }
        }
      }
      if (!valid) raw_lo = raw_hi = make_uint4(0, 0, 0, 0);
      float lo[8], hi[8];
      {
        const uint32_t wl[4] = {raw_lo.x, raw_lo.y, raw_lo.z, raw_lo.w}, wh[4] = {raw_hi.x, raw_hi.y, raw_hi.z, raw_hi.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          lo[2 * i] = __uint_as_float(wl[i] << 16); lo[2 * i + 1] = __uint_as_float(wl[i] & 0xffff0000u);
          hi[2 * i] = __uint_as_float(wh[i] << 16); hi[2 * i + 1] = __uint_as_float(wh[i] & 0xffff0000u);
        }
      }
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) ss += lo[i] * lo[i] + hi[i] * hi[i];
#pragma unroll
      for (int o = L / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (valid && (is_k ? fr.k_gain : fr.q_gain)) {
        const float inv = rsqrtf(ss / (float)D + fr.eps);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          lo[i] = rnd<bf16>(rnd<bf16>(lo[i] * inv) * gq_lo[i]);
          hi[i] = rnd<bf16>(rnd<bf16>(hi[i] * inv) * gq_hi[i]);
        }
      }
      if (valid && fr.cos_table) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float c = rnd<bf16>(cs[i]), s_ = rnd<bf16>(sn[i]);
          const float a = rnd<bf16>(rnd<bf16>(lo[i] * c) + rnd<bf16>(-hi[i] * s_));
          const float b = rnd<bf16>(rnd<bf16>(hi[i] * c) + rnd<bf16>(lo[i] * s_));
          lo[i] = a;
          hi[i] = b;
        }
      }
      const uint4 out_lo = make_uint4(pack_bf16(lo[0], lo[1]), pack_bf16(lo[2], lo[3]), pack_bf16(lo[4], lo[5]), pack_bf16(lo[6], lo[7]));
      const uint4 out_hi = make_uint4(pack_bf16(hi[0], hi[1]), pack_bf16(hi[2], hi[3]), pack_bf16(hi[4], hi[5]), pack_bf16(hi[6], hi[7]));
      if (item < DM_ROWS) {
        *reinterpret_cast<uint4*>(q_tile + tile_offset<D>(item, part)) = out_lo;
        *reinterpret_cast<uint4*>(q_tile + tile_offset<D>(item, part + C / 2)) = out_hi;
      } else if (is_k && valid) {
        *reinterpret_cast<uint4*>(&new_kv[0][part * 8]) = out_lo;
        *reinterpret_cast<uint4*>(&new_kv[0][HALF + part * 8]) = out_hi;
      }
    }
    if (patch && tid < C)
      *reinterpret_cast<uint4*>(&new_kv[1][tid * 8]) =
          *reinterpret_cast<const uint4*>(in_row + (size_t)(heads + kv_heads + kvh) * D + tid * 8);
  }
  __syncthreads();  // the query tile is written (and the new key and value)
  if (FUSED && patch && blockIdx.y % chunks == 0 && tid < 2 * C) {
    // for the steps to come; this step's blocks all patch their own copy instead of reading it back
    const size_t at = page_row(pages[end_page - 1], kvh, pos % SB_PAGE_TOKENS, kv_heads, D) + (size_t)(tid % C) * 8;
    bf16* store = const_cast<bf16*>(tid < C ? k_store : v_store);
    *reinterpret_cast<uint4*>(store + at) = *reinterpret_cast<const uint4*>(&new_kv[tid < C ? 0 : 1][(tid % C) * 8]);
  }

  uint32_t qf[KSTEPS][4];
  {
    const int r = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk)
      ldmatrix_x4(smem_u32(q_tile + tile_offset<D>(r, 2 * kk + (lane >> 4))), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
  }
  float o[NBLK][4];
#pragma unroll
  for (int n = 0; n < NBLK; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

  for (int i = 0; i < n_pages; ++i) {
    load_page(i + DM_STAGES - 1);     // its stage was released by the barrier that ended page i - 1
    cp_wait<DM_STAGES - 1>();         // page i has landed (for this thread's copies)
    __syncthreads();                  // ... and for everyone's
    const uint8_t* kt = ring + (size_t)(i % DM_STAGES) * STAGE_BYTES;
    const uint8_t* vt = kt + PAGE_BYTES;
    if (FUSED && patch && i == n_pages - 1) {
      // the newest position's key and value are not in the cache yet (or only just): use our own
      if (tid < 2 * C) {
        const int in_page = (kv_len - 1) % SB_PAGE_TOKENS;
        uint8_t* tile = const_cast<uint8_t*>(tid < C ? kt : vt);
        *reinterpret_cast<uint4*>(tile + tile_offset<D>(in_page, tid % C)) =
            *reinterpret_cast<const uint4*>(&new_kv[tid < C ? 0 : 1][(tid % C) * 8]);
      }
      __syncthreads();
    }
    const int j0 = (p_begin + i) * SB_PAGE_TOKENS + warp * 16;   // this warp's 16 keys

    float s[2][4];
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
      uint32_t b0, b1, b2, b3;
      const int key = warp * 16 + (lane & 7) + (lane >> 4) * 8;
      ldmatrix_x4(smem_u32(kt + tile_offset<D>(key, 2 * kk + ((lane >> 3) & 1))), b0, b1, b2, b3);
      mma_bf16(s[0], qf[kk], b0, b1);
      mma_bf16(s[1], qf[kk], b2, b3);
    }
    const bool edge = j0 < first || j0 + 16 > kv_len;
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int nb = 0; nb < 2; ++nb) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = s[nb][e] * scale_log2;
        if (edge) {
          const int j = j0 + nb * 8 + (lane & 3) * 2 + (e & 1);
          if (j < first || j >= kv_len) v = -INFINITY;
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
    uint32_t pf[4];
    {
      const float p00 = exp2f(s[0][0] - m_use[0]), p01 = exp2f(s[0][1] - m_use[0]);
      const float p02 = exp2f(s[0][2] - m_use[1]), p03 = exp2f(s[0][3] - m_use[1]);
      const float p10 = exp2f(s[1][0] - m_use[0]), p11 = exp2f(s[1][1] - m_use[0]);
      const float p12 = exp2f(s[1][2] - m_use[1]), p13 = exp2f(s[1][3] - m_use[1]);
      l_run[0] = l_run[0] * alpha[0] + (p00 + p01 + p10 + p11);
      l_run[1] = l_run[1] * alpha[1] + (p02 + p03 + p12 + p13);
      pf[0] = pack_bf16(p00, p01); pf[1] = pack_bf16(p02, p03);
      pf[2] = pack_bf16(p10, p11); pf[3] = pack_bf16(p12, p13);
    }
#pragma unroll
    for (int n = 0; n < NBLK; n += 2) {
      o[n][0] *= alpha[0]; o[n][1] *= alpha[0]; o[n][2] *= alpha[1]; o[n][3] *= alpha[1];
      o[n + 1][0] *= alpha[0]; o[n + 1][1] *= alpha[0]; o[n + 1][2] *= alpha[1]; o[n + 1][3] *= alpha[1];
      uint32_t b0, b1, b2, b3;
      const int key = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
      ldmatrix_x4_trans(smem_u32(vt + tile_offset<D>(key, n + (lane >> 4))), b0, b1, b2, b3);
      mma_bf16(o[n], pf, b0, b1);
      mma_bf16(o[n + 1], pf, b2, b3);
    }
    __syncthreads();  // everyone is done with this stage; the next iteration refills it
  }
  cp_wait<0>();
  __syncthreads();

  // ---- merge the four warps (each saw different keys) through shared memory
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 1);
    l_run[h] += __shfl_xor_sync(0xffffffffu, l_run[h], 2);
  }
  // [warps][16][DP] floats in the ring, which is free now; rows are padded by 8 floats so that the
  // rows a warp stores at once fall into different banks; rows past the group are not stored
  constexpr int DP = D + 8;
  float* sh_o = reinterpret_cast<float*>(ring);
  const int r_a = lane >> 2;
  if ((lane & 3) == 0) {
    sh_m[warp][r_a] = m_run[0]; sh_m[warp][r_a + 8] = m_run[1];
    sh_l[warp][r_a] = l_run[0]; sh_l[warp][r_a + 8] = l_run[1];
  }
  {
    float* base = sh_o + ((size_t)warp * DM_ROWS) * DP;
    const int col0 = (lane & 3) * 2;
    if (r_a < gc) {
#pragma unroll
      for (int n = 0; n < NBLK; ++n)
        *reinterpret_cast<float2*>(base + (size_t)r_a * DP + n * 8 + col0) = make_float2(o[n][0], o[n][1]);
    }
    if (r_a + 8 < gc) {
#pragma unroll
      for (int n = 0; n < NBLK; ++n)
        *reinterpret_cast<float2*>(base + (size_t)(r_a + 8) * DP + n * 8 + col0) = make_float2(o[n][2], o[n][3]);
    }
  }
  __syncthreads();
  for (int idx = tid; idx < gc * D; idx += DM_THREADS) {
    const int r = idx / D, d = idx - r * D;
    float m_all = -INFINITY;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) m_all = fmaxf(m_all, sh_m[w][r]);
    float lsum = 0.f, a = 0.f;
#pragma unroll
    for (int w = 0; w < DM_WARPS; ++w) {
      const float wgt = sh_m[w][r] == -INFINITY ? 0.f : exp2f(sh_m[w][r] - m_all);
      lsum += sh_l[w][r] * wgt;
      a += sh_o[((size_t)w * DM_ROWS + r) * DP + d] * wgt;
    }
    const int head = kvh * groups + g0 + r;
    if (n_splits == 1) {
      out[((size_t)row * heads + head) * D + d] = __float2bfloat16_rn(a / lsum);
    } else if (CLUSTER) {
      sh_o[(size_t)r * DP + d] = a;     // warp 0's place: (r, d) is read by this thread alone
      if (d == 0) { cl_m[r] = m_all; cl_l[r] = lsum; }
    } else {
      const size_t slot = ((size_t)row * heads + head) * n_splits + split;
      part_acc[slot * D + d] = a;
      if (d == 0) { part_ml[slot * 2] = m_all; part_ml[slot * 2 + 1] = lsum; }
    }
  }
  if (CLUSTER && n_splits > 1) {
    // out = sum_s w_s acc_s / sum_s w_s l_s with w_s = 2^(m_s - max m), each block a share of (r, d)
    cluster_sync();
    const uint32_t acc_addr = smem_u32(sh_o), m_addr = smem_u32(cl_m), l_addr = smem_u32(cl_l);
    for (int idx = split * DM_THREADS + tid; idx < gc * D; idx += n_splits * DM_THREADS) {
      const int r = idx / D, d = idx - r * D;
      // all parts' values first (the remote loads are in flight together), then the arithmetic
      float ms[DM_CLUSTER_MAX], ls[DM_CLUSTER_MAX], as[DM_CLUSTER_MAX];
#pragma unroll
      for (int sp = 0; sp < DM_CLUSTER_MAX; ++sp) {
        if (sp < n_splits) {
          ms[sp] = cluster_load(cluster_addr(m_addr + r * 4, sp));
          ls[sp] = cluster_load(cluster_addr(l_addr + r * 4, sp));
          as[sp] = cluster_load(cluster_addr(acc_addr + (r * DP + d) * 4, sp));
        }
      }
      float m_all = -INFINITY;
#pragma unroll
      for (int sp = 0; sp < DM_CLUSTER_MAX; ++sp)
        if (sp < n_splits) m_all = fmaxf(m_all, ms[sp]);
      float lsum = 0.f, a = 0.f;
#pragma unroll
      for (int sp = 0; sp < DM_CLUSTER_MAX; ++sp) {
        if (sp < n_splits && ms[sp] != -INFINITY) {
          const float wgt = exp2f(ms[sp] - m_all);
          lsum += ls[sp] * wgt;
          a += as[sp] * wgt;
        }
      }
      out[((size_t)row * heads + kvh * groups + g0 + r) * D + d] = __float2bfloat16_rn(a / lsum);
    }
    cluster_rendezvous();               // nobody leaves while its shared memory is still read
  }
}

// out[row, head, :] = sum_s w_s acc_s / sum_s w_s l_s with w_s = 2^(m_s - max m)
__global__ void attention_merge_mma_kernel(const float* __restrict__ part_acc,
                                           const float* __restrict__ part_ml, bf16* __restrict__ out,
                                           int n_splits, int head_dim) {
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(part_acc);
  SB_BEHIND_WAIT(part_ml);
  const size_t rh = blockIdx.x;
  float m_all = -INFINITY;
  for (int s = 0; s < n_splits; ++s) m_all = fmaxf(m_all, part_ml[(rh * n_splits + s) * 2]);
  float lsum = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = part_ml[(rh * n_splits + s) * 2];
    if (ms != -INFINITY) lsum += part_ml[(rh * n_splits + s) * 2 + 1] * exp2f(ms - m_all);
  }
  for (int d = threadIdx.x; d < head_dim; d += blockDim.x) {
    float a = 0.f;
    for (int s = 0; s < n_splits; ++s) {
      const float ms = part_ml[(rh * n_splits + s) * 2];
      if (ms != -INFINITY) a += part_acc[(rh * n_splits + s) * head_dim + d] * exp2f(ms - m_all);
    }
    out[rh * head_dim + d] = __float2bfloat16_rn(a / lsum);
  }
}

template <int D, bool FUSED>
static int launch_any(const void* q, void* out, const void* k_store, const void* v_store,
                      const int* block_table, int table_stride, const int* row_slot, const int* row_kv_len,
                      int rows, int heads, int kv_heads, float scale, int window, int n_splits,
                      float* part_acc, float* part_ml, const FusedRope& fr, cudaStream_t s) {
  // queries + ring; the ring is reused for the warps' float partial results at the end
  constexpr int RING = DM_STAGES * 2 * SB_PAGE_TOKENS * D * 2;
  constexpr int MERGE = DM_WARPS * DM_ROWS * (D + 8) * 4;
  const int smem = DM_ROWS * D * 2 + (RING > MERGE ? RING : MERGE);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_mma_kernel<D, false, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(attention_decode_mma_kernel<D, true, FUSED>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int groups = heads / kv_heads;
  const int chunks = (groups + DM_ROWS - 1) / DM_ROWS;
  dim3 grid(rows, kv_heads * chunks, n_splits);
  if (n_splits > 1 && n_splits <= DM_CLUSTER_MAX)
    return launch_dependent_cluster(attention_decode_mma_kernel<D, true, FUSED>, grid, dim3(DM_THREADS), smem, s,
        dim3(1, 1, n_splits), (const bf16*)q, (bf16*)out, (const bf16*)k_store, (const bf16*)v_store,
        block_table, table_stride, row_slot, row_kv_len, heads, kv_heads, scale * 1.4426950408889634f,
        window, n_splits, part_acc, part_ml, fr);
  int rc = launch_dependent(attention_decode_mma_kernel<D, false, FUSED>, grid, dim3(DM_THREADS), smem, s,
      (const bf16*)q, (bf16*)out, (const bf16*)k_store, (const bf16*)v_store, block_table, table_stride,
      row_slot, row_kv_len, heads, kv_heads, scale * 1.4426950408889634f, window, n_splits, part_acc,
      part_ml, fr);
  if (rc || n_splits == 1) return rc;
  return launch_dependent(attention_merge_mma_kernel, dim3(rows * heads), dim3(D < 128 ? D : 128), 0, s,
                          (const float*)part_acc, (const float*)part_ml, (bf16*)out, n_splits, D);
}

template <int D>
static int launch(const void* q, void* out, const void* k_store, const void* v_store,
                  const int* block_table, int table_stride, const int* row_slot, const int* row_kv_len,
                  int rows, int heads, int kv_heads, float scale, int window, int n_splits,
                  float* part_acc, float* part_ml, cudaStream_t s) {
  FusedRope none = {};
  return launch_any<D, false>(q, out, k_store, v_store, block_table, table_stride, row_slot, row_kv_len, rows,
                              heads, kv_heads, scale, window, n_splits, part_acc, part_ml, none, s);
}

extern "C" {

// Same contract as sb_attention_decode, bfloat16 only; head_dim 16, 32, 64 or 128 (-2 otherwise).
int sb_attention_decode_mma(const void* q, void* out, const void* k_store, const void* v_store,
                            const int* block_table, int table_stride, const int* row_slot,
                            const int* row_kv_len, int rows, int heads, int kv_heads, int head_dim,
                            float scale, int window, int n_splits, float* part_acc, float* part_ml,
                            cudaStream_t s) {
  if (rows == 0) return 0;
  if (kv_heads <= 0 || heads % kv_heads || n_splits < 1) return -2;
#define ARGS q, out, k_store, v_store, block_table, table_stride, row_slot, row_kv_len, rows, heads, \
             kv_heads, scale, window, n_splits, part_acc, part_ml, s
  switch (head_dim) {
    case 16: return launch<16>(ARGS);
    case 32: return launch<32>(ARGS);
    case 64: return launch<64>(ARGS);
    case 128: return launch<128>(ARGS);
    default: return -2;
  }
#undef ARGS
}

// The same for a one-token step straight from the q/k/v product: qkv [rows, q_stride] bfloat16 holds
// the query heads and, if has_kv, behind them the key and the value heads of each row's new token
// (position row_kv_len - 1).  Head norm (gains may be null; gain_dtype 0 float, 1 bfloat16), rotation
// (tables [positions, head_dim / 2] float, may be null) and, if has_kv, the cache write happen here.
// early: see the kernel (only with has_kv: a layer that reads another layer's cache must wait).
int sb_attention_decode_mma_fused(const void* qkv, int q_stride, void* out, void* k_store, void* v_store,
                                  const int* block_table, int table_stride, const int* row_slot,
                                  const int* row_kv_len, int rows, int heads, int kv_heads, int head_dim,
                                  float scale, int window, int n_splits, float* part_acc, float* part_ml,
                                  const void* q_gain, const void* k_gain, int gain_dtype, float eps,
                                  const float* cos_table, const float* sin_table, int has_kv, int early,
                                  cudaStream_t s) {
  if (rows == 0) return 0;
  if (kv_heads <= 0 || heads % kv_heads || n_splits < 1) return -2;
  if (q_stride % 8 || (((uintptr_t)qkv | (uintptr_t)k_store | (uintptr_t)v_store) & 15)) return -2;
  if ((cos_table == nullptr) != (sin_table == nullptr)) return -2;
  FusedRope fr;
  fr.q_stride = q_stride; fr.has_kv = has_kv; fr.gain_f32 = gain_dtype == 0; fr.eps = eps;
  fr.q_gain = q_gain; fr.k_gain = k_gain; fr.cos_table = cos_table; fr.sin_table = sin_table;
  fr.early = early && has_kv;
#define ARGS qkv, out, k_store, v_store, block_table, table_stride, row_slot, row_kv_len, rows, heads, \
             kv_heads, scale, window, n_splits, part_acc, part_ml, fr, s
  switch (head_dim) {
    case 16: return launch_any<16, true>(ARGS);
    case 32: return launch_any<32, true>(ARGS);
    case 64: return launch_any<64, true>(ARGS);
    case 128: return launch_any<128, true>(ARGS);
    default: return -2;
  }
#undef ARGS
}

}  // extern "C"
