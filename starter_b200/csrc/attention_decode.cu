// Single-token attention over the paged cache, split over the keys so that one long sequence fills
// the GPU (engine/kernels/fused.py:729-823), with the query heads that share a key/value head handled
// together so each key and value is read once (fused.py:641-709).
//
// Grid (row, kv_head * head_chunks, split).  A page of one key/value head is one contiguous block of
// 64 x head_dim elements, so a producer warp brings whole pages into a ring of shared-memory stages
// with bulk asynchronous copies (cp.async.bulk, completion on an mbarrier) while four consumer warps
// work on the pages that have landed: many kilobytes per SM are in flight whatever the occupancy.
// Inside a page the warps take keys in turn, and inside a warp head_dim / 16 lanes share one key
// (16 elements each).  Every such lane group keeps its own running maximum, sum and accumulator in
// float (fused.py:288-312); groups, warps and finally splits are merged by rescaling onto the common
// maximum, and a part that saw no key drops out (fused.py:793-823).  Lengths come from device memory,
// so one captured launch serves every step (fused.py:262-271), and they are per row.  A query at
// position p sees keys first..p, first = max(0, p + 1 - window).
//
// Every wait on an mbarrier gives up after WAIT_LIMIT_NS, raises bit 8 of *status and lets the block
// drain and return.
#include "common.cuh"

#define AD_WARPS 4
#define AD_MAXG 4
#define AD_ELEMS 16
#define AD_THREADS ((AD_WARPS + 1) * 32)
#define AD_MAX_STAGES 4
#define AD_RING_BYTES (96 * 1024)
#define WAIT_LIMIT_NS 2000000000ull

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t now_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort,
                                          uint64_t limit_ns = WAIT_LIMIT_NS) {
  if (mbar_try(bar, parity)) return true;
  const uint64_t start = now_ns();
  while (true) {
    if (mbar_try(bar, parity)) return true;
    if (*abort) return false;
    if (now_ns() - start > limit_ns) { *abort = 1; return false; }
  }
}

// One contiguous run of bytes (a multiple of 16, 16-byte aligned on both sides) into shared memory.
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
      ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

template <typename T> __device__ __forceinline__ void load16(const T* p, float* out);
template <> __device__ __forceinline__ void load16<bf16>(const bf16* p, float* out) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  const uint4 b = *reinterpret_cast<const uint4*>(p + 8);
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
template <> __device__ __forceinline__ void load16<float>(const float* p, float* out) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float4 v = *reinterpret_cast<const float4*>(p + 4 * i);
    out[4 * i] = v.x; out[4 * i + 1] = v.y; out[4 * i + 2] = v.z; out[4 * i + 3] = v.w;
  }
}

template <typename T, int D> struct DecodeShape {
  static constexpr int PAGE_BYTES = SB_PAGE_TOKENS * D * (int)sizeof(T);   // keys (or values) of a page
  static constexpr int STAGE_BYTES = 2 * PAGE_BYTES;
  static constexpr int FIT = AD_RING_BYTES / STAGE_BYTES;
  static constexpr int STAGES = FIT > AD_MAX_STAGES ? AD_MAX_STAGES : (FIT < 2 ? 2 : FIT);
  static constexpr int RING_BYTES = STAGES * STAGE_BYTES;
};

template <typename T, int D>
__global__ void __launch_bounds__(AD_THREADS)
attention_decode_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ k_store,
                        const T* __restrict__ v_store, const int* __restrict__ block_table,
                        int table_stride, const int* __restrict__ row_slot,
                        const int* __restrict__ row_kv_len, int heads, int kv_heads, float scale_log2,
                        int window, int n_splits, float* __restrict__ part_acc,
                        float* __restrict__ part_ml, int* status, unsigned long long limit_ns,
                        int withhold_page) {
  using Shape = DecodeShape<T, D>;
  constexpr int LPK = D / AD_ELEMS;  // lanes that share a key
  constexpr int KPW = 32 / LPK;      // keys a warp takes at a time
  constexpr int STAGES = Shape::STAGES;
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ float sh_acc[AD_WARPS][AD_MAXG][D];
  __shared__ float sh_m[AD_WARPS][AD_MAXG];
  __shared__ float sh_l[AD_WARPS][AD_MAXG];
  __shared__ uint64_t full_bar[STAGES], empty_bar[STAGES];
  __shared__ int abort_flag;

  const int groups = heads / kv_heads;
  const int chunks = (groups + AD_MAXG - 1) / AD_MAXG;
  const int row = blockIdx.x;
  const int kvh = blockIdx.y / chunks;
  const int g0 = (blockIdx.y % chunks) * AD_MAXG;
  const int gc = min(AD_MAXG, groups - g0);
  const int split = blockIdx.z;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int part = lane % LPK, sub = lane / LPK;

  const int kv_len = row_kv_len[row];
  int first = 0;
  if (window > 0 && kv_len - window > 0) first = kv_len - window;
  const int first_page = first / SB_PAGE_TOKENS;
  const int end_page = (kv_len + SB_PAGE_TOKENS - 1) / SB_PAGE_TOKENS;
  const int per_split = (end_page - first_page + n_splits - 1) / n_splits;
  const int p_begin = first_page + split * per_split;
  const int p_end = min(p_begin + per_split, end_page);
  const int n_pages = max(p_end - p_begin, 0);
  const int* pages = block_table + (size_t)row_slot[row] * table_stride;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], AD_WARPS); }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  volatile int* abort = &abort_flag;

  if (warp == AD_WARPS) {
    // ---------------- producer: one lane streams the pages of this split into the ring
    if (lane == 0) {
      int issued = 0;
      for (int i = 0; i < n_pages; ++i) {
        const int s = i % STAGES;
        if (i >= STAGES && !mbar_wait(&empty_bar[s], ((i / STAGES) - 1) & 1, abort, limit_ns)) break;
        const size_t base = page_row(pages[p_begin + i], kvh, 0, kv_heads, D);
        uint8_t* dst = ring + (size_t)s * Shape::STAGE_BYTES;
        mbar_expect_tx(&full_bar[s], Shape::STAGE_BYTES);
        bulk_load(dst, k_store + base, Shape::PAGE_BYTES, &full_bar[s]);
        // (tests of the give-up path leave one page's values out: its stage then never completes)
        if (i != withhold_page)
          bulk_load(dst + Shape::PAGE_BYTES, v_store + base, Shape::PAGE_BYTES, &full_bar[s]);
        issued = i + 1;
      }
      if (*abort) {
        for (int i = max(issued - STAGES, 0); i < issued; ++i) {
          const uint64_t start = now_ns();
          while (!mbar_try(&full_bar[i % STAGES], (i / STAGES) & 1) && now_ns() - start < limit_ns) {}
        }
      }
    }
  } else {
    // ---------------- consumers
    float qv[AD_MAXG][AD_ELEMS], acc[AD_MAXG][AD_ELEMS], m[AD_MAXG], l[AD_MAXG];
#pragma unroll
    for (int g = 0; g < AD_MAXG; ++g) {
      m[g] = -INFINITY;
      l[g] = 0.f;
#pragma unroll
      for (int i = 0; i < AD_ELEMS; ++i) acc[g][i] = 0.f;
      if (g < gc) {
        load16<T>(q + ((size_t)row * heads + (size_t)kvh * groups + g0 + g) * D + part * AD_ELEMS, qv[g]);
#pragma unroll
        for (int i = 0; i < AD_ELEMS; ++i) qv[g][i] *= scale_log2;
      } else {
#pragma unroll
        for (int i = 0; i < AD_ELEMS; ++i) qv[g][i] = 0.f;
      }
    }

    for (int i = 0; i < n_pages; ++i) {
      const int s = i % STAGES;
      if (!mbar_wait(&full_bar[s], (i / STAGES) & 1, abort, limit_ns)) break;
      const T* kp = reinterpret_cast<const T*>(ring + (size_t)s * Shape::STAGE_BYTES);
      const T* vp = reinterpret_cast<const T*>(ring + (size_t)s * Shape::STAGE_BYTES + Shape::PAGE_BYTES);
      const int p = p_begin + i;
#pragma unroll 2
      for (int k0 = warp * KPW; k0 < SB_PAGE_TOKENS; k0 += AD_WARPS * KPW) {
        const int in_page = k0 + sub;
        const int j = p * SB_PAGE_TOKENS + in_page;
        const bool valid = j >= first && j < kv_len;
        float kx[AD_ELEMS], vx[AD_ELEMS];
        load16<T>(kp + (size_t)in_page * D + part * AD_ELEMS, kx);
        load16<T>(vp + (size_t)in_page * D + part * AD_ELEMS, vx);
#pragma unroll
        for (int g = 0; g < AD_MAXG; ++g) {
          if (g < gc) {
            float sc = 0.f;
#pragma unroll
            for (int e = 0; e < AD_ELEMS; ++e) sc += qv[g][e] * kx[e];
#pragma unroll
            for (int o = LPK / 2; o > 0; o >>= 1) sc += __shfl_xor_sync(0xffffffffu, sc, o);
            if (valid) {
              const float m_new = fmaxf(m[g], sc);
              const float alpha = exp2f(m[g] - m_new);
              const float pr = exp2f(sc - m_new);
              l[g] = l[g] * alpha + pr;
#pragma unroll
              for (int e = 0; e < AD_ELEMS; ++e) acc[g][e] = acc[g][e] * alpha + pr * vx[e];
              m[g] = m_new;
            }
          }
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }

    // merge the lane groups of a warp (same `part`, different `sub`)
#pragma unroll
    for (int g = 0; g < AD_MAXG; ++g) {
      float m_all = m[g];
#pragma unroll
      for (int o = LPK; o < 32; o <<= 1) m_all = fmaxf(m_all, __shfl_xor_sync(0xffffffffu, m_all, o));
      const float w = m[g] == -INFINITY ? 0.f : exp2f(m[g] - m_all);
      float lsum = l[g] * w;
#pragma unroll
      for (int o = LPK; o < 32; o <<= 1) lsum += __shfl_xor_sync(0xffffffffu, lsum, o);
#pragma unroll
      for (int e = 0; e < AD_ELEMS; ++e) {
        float a = acc[g][e] * w;
#pragma unroll
        for (int o = LPK; o < 32; o <<= 1) a += __shfl_xor_sync(0xffffffffu, a, o);
        acc[g][e] = a;
      }
      if (sub == 0) {
#pragma unroll
        for (int e = 0; e < AD_ELEMS; ++e) sh_acc[warp][g][part * AD_ELEMS + e] = acc[g][e];
        if (part == 0) { sh_m[warp][g] = m_all; sh_l[warp][g] = lsum; }
      }
    }
  }
  __syncthreads();

  // merge the warps; thread t finishes elements t, t + 128, ... of each head
  if (warp < AD_WARPS && !abort_flag) {
    for (int idx = threadIdx.x; idx < gc * D; idx += AD_WARPS * 32) {
      const int g = idx / D, d = idx - g * D;
      float m_all = -INFINITY;
#pragma unroll
      for (int w = 0; w < AD_WARPS; ++w) m_all = fmaxf(m_all, sh_m[w][g]);
      float lsum = 0.f, a = 0.f;
#pragma unroll
      for (int w = 0; w < AD_WARPS; ++w) {
        const float wgt = sh_m[w][g] == -INFINITY ? 0.f : exp2f(sh_m[w][g] - m_all);
        lsum += sh_l[w][g] * wgt;
        a += sh_acc[w][g][d] * wgt;
      }
      const int head = kvh * groups + g0 + g;
      if (n_splits == 1) {
        out[((size_t)row * heads + head) * D + d] = from_f<T>(a / lsum);
      } else {
        const size_t slot = ((size_t)row * heads + head) * n_splits + split;
        part_acc[slot * D + d] = a;
        if (d == 0) { part_ml[slot * 2] = m_all; part_ml[slot * 2 + 1] = lsum; }
      }
    }
  }
  if (threadIdx.x == 0 && abort_flag && status) atomicOr(status, 8);
}

// out[row, head, :] = sum_s w_s acc_s / sum_s w_s l_s with w_s = 2^(m_s - max m)
template <typename T>
__global__ void attention_merge_kernel(const float* __restrict__ part_acc,
                                       const float* __restrict__ part_ml, T* __restrict__ out,
                                       int n_splits, int head_dim) {
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
    out[rh * head_dim + d] = from_f<T>(a / lsum);
  }
}

// Set by sb_attention_decode_withhold for the next launch only (tests of the give-up path).
static unsigned long long next_limit_ns = WAIT_LIMIT_NS;
static int next_withhold_page = -1;

template <typename T, int D>
static int launch(const void* q, void* out, const void* k_store, const void* v_store,
                  const int* block_table, int table_stride, const int* row_slot, const int* row_kv_len,
                  int rows, int heads, int kv_heads, float scale, int window, int n_splits,
                  float* part_acc, float* part_ml, int* status, cudaStream_t s) {
  using Shape = DecodeShape<T, D>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_decode_kernel<T, D>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, Shape::RING_BYTES);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  const int groups = heads / kv_heads;
  const int chunks = (groups + AD_MAXG - 1) / AD_MAXG;
  dim3 grid(rows, kv_heads * chunks, n_splits);
  attention_decode_kernel<T, D><<<grid, AD_THREADS, Shape::RING_BYTES, s>>>(
      (const T*)q, (T*)out, (const T*)k_store, (const T*)v_store, block_table, table_stride, row_slot,
      row_kv_len, heads, kv_heads, scale * 1.4426950408889634f, window, n_splits, part_acc, part_ml,
      status, next_limit_ns, next_withhold_page);
  next_limit_ns = WAIT_LIMIT_NS;
  next_withhold_page = -1;
  int rc = SB_LAUNCH_RESULT();
  if (rc || n_splits == 1) return rc;
  attention_merge_kernel<T><<<rows * heads, D < 128 ? D : 128, 0, s>>>(part_acc, part_ml, (T*)out,
                                                                      n_splits, D);
  return SB_LAUNCH_RESULT();
}

extern "C" {

// For tests of the give-up path: the NEXT sb_attention_decode launch leaves out the values of page
// `page` of every block's range (blocks with fewer pages are unaffected) and its waits give up after
// `limit_ns`.  That launch cannot finish its sums; it must return with bit 8 of *status set.
void sb_attention_decode_withhold(int page, unsigned long long limit_ns) {
  next_withhold_page = page;
  next_limit_ns = limit_ns ? limit_ns : WAIT_LIMIT_NS;
}

// q, out: [rows, heads * head_dim]; one query per row at position row_kv_len[row] - 1 of the sequence
// in slot row_slot[row].  part_acc [rows * heads * n_splits * head_dim] and part_ml
// [rows * heads * n_splits * 2] floats are scratch, unused when n_splits == 1.
// head_dim must be 16, 32, 64, 128 or 256 (returns -2 otherwise).
int sb_attention_decode(int dtype, const void* q, void* out, const void* k_store, const void* v_store,
                        const int* block_table, int table_stride, const int* row_slot,
                        const int* row_kv_len, int rows, int heads, int kv_heads, int head_dim,
                        float scale, int window, int n_splits, float* part_acc, float* part_ml,
                        int* status, cudaStream_t s) {
  if (rows == 0) return 0;
  if (kv_heads <= 0 || heads % kv_heads || n_splits < 1) return -2;
#define ARGS q, out, k_store, v_store, block_table, table_stride, row_slot, row_kv_len, rows, heads, \
             kv_heads, scale, window, n_splits, part_acc, part_ml, status, s
#define BY_DTYPE(D)                                   \
  if (dtype == 0) return launch<float, D>(ARGS);      \
  if (dtype == 1) return launch<bf16, D>(ARGS);       \
  return -1;
  switch (head_dim) {
    case 16: BY_DTYPE(16)
    case 32: BY_DTYPE(32)
    case 64: BY_DTYPE(64)
    case 128: BY_DTYPE(128)
    case 256: BY_DTYPE(256)
    default: return -2;
  }
#undef BY_DTYPE
#undef ARGS
}

}  // extern "C"
