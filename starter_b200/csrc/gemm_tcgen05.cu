// y[m, n] = sum_k x[m, k] * w[n, k] in bfloat16 on the fifth-generation tensor cores.
//
// The weight matrix is the streamed operand: a CTA owns 128 weight rows (the MMA's M) and up to 256
// activation rows (the MMA's N), so the same kernel serves one decode row and a prompt.  TMA brings
// [64 x 64] boxes of w and a [BM x 64] box of x into a ring of shared-memory stages (128-byte
// swizzle, K-major); one thread issues tcgen05.mma (kind::f16, float accumulation in tensor memory);
// four warps read the accumulator back with tcgen05.ld and write the result.  Rows past the end of
// either matrix are zero-filled by TMA and masked on the way out, so no size needs padding.
//
// For a few rows the product is bound by reading w, and 128-row tiles alone would leave most SMs idle
// (a 2560-row projection has 20), so the k range is cut into up to 8 `splits` that run as the CTAs of
// one thread-block cluster.  Each CTA leaves its float partial tile in its own shared memory; after
// a cluster barrier every CTA adds, for its share of the tile, the parts of all CTAs in split order
// through distributed shared memory (so the sum does not depend on timing,
// engine/kernels/fused.py:474-476) and applies the epilogue.  Nothing goes through global memory.
//
// With `gated`, w is [gate; up] stacked ([2 * n_out, k]); a tile holds 64 gate rows and the matching
// 64 up rows and the epilogue writes round(silu(gate)) * up (fused.py:89-112).
//
// Every wait on an mbarrier gives up after a time limit (WAIT_LIMIT_NS unless the caller gives one),
// raises bit 4 of *status and lets the CTA drain, free its tensor memory and return.  So that this
// path can be exercised without a fault, the entry point sb_gemm_tcgen05_withheld leaves out one
// activation copy on purpose: the stage it belongs to never completes, the wait on it runs out and
// the kernel must come back with the status bit set.
#include "tcgen05.cuh"
#include "tensor_map.cuh"

#define TILE_N 128      // weight rows per CTA (MMA M)
#define TILE_K 64       // k per stage: 128 bytes of bfloat16, one swizzle atom
#define HALF_BYTES (64 * TILE_K * 2)
#define A_BYTES (2 * HALF_BYTES)
#define GEMM_THREADS 192
#define GEMM_MAX_STAGES 8
#define GEMM_MAX_SPLITS 8
#define WAIT_LIMIT_NS TC_WAIT_LIMIT_NS

// ------------------------------------------------------------------------------------------ kernel

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address, in the cluster's shared window, of `addr` (an address of this CTA) in CTA `rank`.
__device__ __forceinline__ uint32_t in_cta(uint32_t addr, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(addr), "r"(rank));
  return a;
}
__device__ __forceinline__ float ld_cluster(uint32_t addr) {
  float v;
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float4 ld_cluster4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
// The same without publishing anything: a rendezvous only.  (A releasing arrive first waits for this
// thread's earlier global stores to be performed, about a microsecond after the output is written.)
__device__ __forceinline__ void cluster_rendezvous() {
  asm volatile("barrier.cluster.arrive.relaxed;\n\tbarrier.cluster.wait;" ::: "memory");
}

struct GemmArgs {
  void* out;            // [rows, n_out] bfloat16 or float
  int* status;
  int rows, n_out, k_dim;
  int splits, stages, gated, out_float;
  unsigned long long wait_limit_ns;   // how long a wait may take before the CTA gives up
  int withhold_stage;                 // >= 0: the activation copy of this k-block is left out (tests)
};

template <int BM, bool GATED>
__global__ void __launch_bounds__(GEMM_THREADS)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                    const GemmArgs args) {
  constexpr int B_BYTES = BM * TILE_K * 2;
  constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  constexpr uint32_t TMEM_COLS = BM < 32 ? 32 : BM;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[GEMM_MAX_STAGES], empty_bar[GEMM_MAX_STAGES], acc_bar;
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  const int STAGES = args.stages;
  const uint64_t limit = args.wait_limit_ns;
  // the warp's number as a value the compiler knows to be the same in every lane
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  const int tile = blockIdx.x, split = blockIdx.y, mtile = blockIdx.z;
  const int m0 = mtile * BM;
  const int kb_total = (args.k_dim + TILE_K - 1) / TILE_K;
  const int kb_per = (kb_total + args.splits - 1) / args.splits;
  const int kb_begin = split * kb_per;
  const int kb_end = min(kb_begin + kb_per, kb_total);
  const int n_kb = max(kb_end - kb_begin, 0);
  // rows of w in the two 64-row halves of the tile
  const int row_a = GATED ? tile * 64 : tile * TILE_N;
  const int row_b = GATED ? args.n_out + tile * 64 : tile * TILE_N + 64;
  const int rows_here = min(BM, args.rows - m0);
  // the result goes straight from tensor memory to global memory unless parts must be added or
  // gate and up rows (held by different threads) must meet
  const bool staged = args.splits > 1 || GATED;
  float* part_sm = reinterpret_cast<float*>(smem);   // [BM][TILE_N] floats, in the idle ring

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    mbar_init(&acc_bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_trigger();
  if (warp == 1) tmem_alloc(&tmem_holder, TMEM_COLS);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = tmem_holder;
  volatile int* abort = &abort_flag;

  if (warp == 0) {
    // ---------------- producer: the warp walks the ring together, one elected lane issues the copies.
    // (Role code that only one lane runs, inside a branch on the lane number, is divergent code to the
    // compiler: addresses and descriptors then live in ordinary registers and each TMA or MMA
    // instruction, which wants them in uniform registers, costs over a hundred cycles to issue.
    // Measured on the prompt product: 1170 cycles a k-block that way, 390 this way.)
    const bool elected = elect_one();
    int issued = 0;
    // the weights do not depend on the kernels before this one: the first stages' weight tiles are
    // on their way before the predecessor has finished; the activations follow after the wait
    const int early = min(n_kb, STAGES);
    for (int i = 0; i < early; ++i) {
      uint8_t* a = smem + (size_t)i * STAGE_BYTES;
      const int k = (kb_begin + i) * TILE_K;
      if (elected) {
        mbar_expect_tx(&full_bar[i], STAGE_BYTES);
        tma_load_2d(a, &map_w, &full_bar[i], k, row_a);
        tma_load_2d(a + HALF_BYTES, &map_w, &full_bar[i], k, row_b);
      }
    }
    pdl_wait();
    for (int i = 0; i < early; ++i)
      if (elected && i != args.withhold_stage)
        tma_load_2d(smem + (size_t)i * STAGE_BYTES + A_BYTES, &map_x, &full_bar[i], (kb_begin + i) * TILE_K, m0);
    issued = early;
    int s = 0;
    uint32_t parity = 0;
    for (int i = early; i < n_kb; ++i) {
      if (!__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], parity, abort, limit))) break;
      uint8_t* a = smem + (size_t)s * STAGE_BYTES;
      const int k = (kb_begin + i) * TILE_K;
      if (elected) {
        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
        tma_load_2d(a, &map_w, &full_bar[s], k, row_a);
        tma_load_2d(a + HALF_BYTES, &map_w, &full_bar[s], k, row_b);
        tma_load_2d(a + A_BYTES, &map_x, &full_bar[s], k, m0);
      }
      issued = i + 1;
      if (++s == STAGES) { s = 0; parity ^= 1; }
    }
    if (*abort && elected) {
      // copies still in flight write into this CTA's shared memory: give them time to land
      for (int i = max(issued - STAGES, 0); i < issued; ++i) {
        const uint64_t start = now_ns();
        while (!mbar_try(&full_bar[i % STAGES], (i / STAGES) & 1) && now_ns() - start < limit) {}
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: the warp walks the ring together, one elected lane issues
    const bool elected = elect_one();
    const uint32_t idesc = instr_desc(BM);
    int s = 0;
    uint32_t parity = 0;
    for (int i = 0; i < n_kb; ++i) {
      if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[s], parity, abort, limit))) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
      const uint64_t a_desc = smem_desc(a_addr), b_desc = smem_desc(a_addr + A_BYTES);
      if (elected) {
#pragma unroll
        for (int k = 0; k < TILE_K / 16; ++k) {
          // 16 elements of k are 32 bytes: 2 units of the descriptor's 16-byte address
          umma_bf16(tmem, a_desc + 2 * k, b_desc + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[s]);
      }
      __syncwarp();
      if (++s == STAGES) { s = 0; parity ^= 1; }
    }
    if (elected) umma_commit(&acc_bar);
    __syncwarp();
  } else {
    // ---------------- epilogue, first half: warps 2..5 own the TMEM lane quarters 2, 3, 0, 1
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;                 // row of the tile = TMEM lane
    pdl_wait();   // before the first store: the output may be memory an earlier kernel still reads
    const bool have = n_kb > 0 && mbar_wait(&acc_bar, 0, abort, limit);
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const int n = tile * TILE_N + r;                   // output column when not gated
#pragma unroll 1
    for (int c = 0; c < rows_here; c += 8) {
      float v[8];
      if (have) tmem_load8(tmem + ((uint32_t)(quarter * 32) << 16) + c, v);
      else {
#pragma unroll
        for (int j = 0; j < 8; ++j) v[j] = 0.f;
      }
      if (staged) {
        // column-major, so that consecutive threads write consecutive words
#pragma unroll
        for (int j = 0; j < 8; ++j) part_sm[(c + j) * TILE_N + r] = v[j];
      } else if (n < args.n_out) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const int m = c + j;
          if (m < rows_here) {
            const size_t at = (size_t)(m0 + m) * args.n_out + n;
            if (args.out_float) ((float*)args.out)[at] = v[j];
            else ((bf16*)args.out)[at] = __float2bfloat16_rn(v[j]);
          }
        }
      }
    }
  }

  // ---------------- epilogue, second half: add the parts of all splits and finish
  if (staged) {
    if (args.splits > 1) cluster_sync(); else __syncthreads();
    if (warp >= 2 && !*abort) {
      const uint32_t rank = args.splits > 1 ? cluster_rank() : 0;
      const int out_rows = GATED ? 64 : TILE_N;
      const int per_row = out_rows / 4;                 // an item: four neighbouring outputs of a row
      const int n_items = per_row * rows_here;
      const uint32_t base = smem_u32(part_sm);
      uint32_t remote[GEMM_MAX_SPLITS];
#pragma unroll
      for (int s = 0; s < GEMM_MAX_SPLITS; ++s) remote[s] = s < args.splits && args.splits > 1 ? in_cta(base, s) : base;
      const bool vector_store = args.n_out % 4 == 0;
      // blocks of 128 items go round the cluster; the loads of all parts of an item are in flight
      // together and are added in split order
      for (int item = rank * 128 + (threadIdx.x - 64); item < n_items; item += args.splits * 128) {
        const int m = item / per_row;
        const int orow = (item - m * per_row) * 4;
        const uint32_t at_g = (uint32_t)(m * TILE_N + orow) * 4;
        float4 gv[GEMM_MAX_SPLITS], uv[GEMM_MAX_SPLITS];
#pragma unroll
        for (int s = 0; s < GEMM_MAX_SPLITS; ++s) {
          if (s < args.splits) {
            gv[s] = ld_cluster4(remote[s] + at_g);
            if (GATED) uv[s] = ld_cluster4(remote[s] + at_g + 64 * 4);
          }
        }
        float g[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int s = 0; s < GEMM_MAX_SPLITS; ++s) {
          if (s < args.splits) {
            g[0] += gv[s].x; g[1] += gv[s].y; g[2] += gv[s].z; g[3] += gv[s].w;
            if (GATED) { u[0] += uv[s].x; u[1] += uv[s].y; u[2] += uv[s].z; u[3] += uv[s].w; }
          }
        }
        if (GATED) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float gr = rnd<bf16>(g[j]), ur = rnd<bf16>(u[j]);
            g[j] = rnd<bf16>(gr / (1.f + __expf(-gr))) * ur;
          }
        }
        const int ncol = (GATED ? tile * 64 : tile * TILE_N) + orow;
        const size_t at = (size_t)(m0 + m) * args.n_out + ncol;
        if (vector_store && ncol + 3 < args.n_out) {
          if (args.out_float) {
            *reinterpret_cast<float4*>((float*)args.out + at) = make_float4(g[0], g[1], g[2], g[3]);
          } else {
            __nv_bfloat162 lo = __floats2bfloat162_rn(g[0], g[1]), hi = __floats2bfloat162_rn(g[2], g[3]);
            *reinterpret_cast<uint2*>((bf16*)args.out + at) =
                make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
          }
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            if (ncol + j < args.n_out) {
              if (args.out_float) ((float*)args.out)[at + j] = g[j];
              else ((bf16*)args.out)[at + j] = __float2bfloat16_rn(g[j]);
            }
          }
        }
      }
    }
    // nobody leaves (and gives up its shared memory) while a neighbour may still read it; the reads
    // of a thread have returned when it gets here, because its sums needed them
    if (args.splits > 1) cluster_rendezvous();
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) tmem_free(tmem, TMEM_COLS);
  if (threadIdx.x == 0 && abort_flag && args.status) atomicOr(args.status, 4);
}

// ------------------------------------------------------------------------------------------ host

template <int BM, bool GATED>
static int launch(const CUtensorMap& map_w, const CUtensorMap& map_x, const GemmArgs& args, int tiles,
                  int m_tiles, cudaStream_t s) {
  constexpr int STAGE_BYTES = A_BYTES + BM * TILE_K * 2;
  const int smem = args.stages * STAGE_BYTES + 1024;
  if (smem > 227 * 1024 || args.stages * STAGE_BYTES < BM * TILE_N * 4) return -2;
  static int configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_tcgen05_kernel<BM, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  dim3 grid(tiles, args.splits, m_tiles);
  return launch_dependent_cluster(gemm_tcgen05_kernel<BM, GATED>, grid, dim3(GEMM_THREADS), smem, s,
                                  dim3(1, args.splits, 1), map_w, map_x, args);
}

extern "C" {

// x [rows, k_dim] and w [n_out (2 * n_out if gated), k_dim] bfloat16, row-major, 16-byte aligned,
// k_dim a multiple of 8.  bm (16, 32, 64, 128 or 256) is the number of activation rows per tile,
// splits (1..8) the number of CTAs that share a tile's k range, stages (2..8) the depth of the ring;
// stages * (16 KB + bm * 128 B) must hold the bm x 128 float tile and fit in shared memory.
// Returns -2 for sizes it does not take, -3/-4 if the tensor maps cannot be made.
static int gemm_entry(const void* x, const void* w, void* out, int rows, int n_out, int k_dim, int bm,
                      int splits, int stages, int gated, int out_float, int* status,
                      unsigned long long wait_limit_ns, int withhold_stage, cudaStream_t s) {
  if (rows == 0 || n_out == 0) return 0;
  if (k_dim % 8 || k_dim <= 0 || splits < 1 || splits > GEMM_MAX_SPLITS) return -2;
  if (stages < 2 || stages > GEMM_MAX_STAGES) return -2;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return -2;
  if (gated && n_out % 64) return -2;
  const int tiles = gated ? n_out / 64 : (n_out + TILE_N - 1) / TILE_N;
  const int m_tiles = (rows + bm - 1) / bm;
  const int w_rows = gated ? 2 * n_out : n_out;
  CUtensorMap map_w, map_x;
  int rc = sb_make_map(&map_w, w, w_rows, k_dim, 64);
  if (rc) return rc;
  rc = sb_make_map(&map_x, x, rows, k_dim, bm);
  if (rc) return rc;
  GemmArgs args;
  args.out = out; args.status = status;
  args.rows = rows; args.n_out = n_out; args.k_dim = k_dim;
  args.splits = splits; args.stages = stages; args.gated = gated; args.out_float = out_float;
  args.wait_limit_ns = wait_limit_ns; args.withhold_stage = withhold_stage;
#define BY_TILE(G)                                                           \
  switch (bm) {                                                              \
    case 16: return launch<16, G>(map_w, map_x, args, tiles, m_tiles, s);    \
    case 32: return launch<32, G>(map_w, map_x, args, tiles, m_tiles, s);    \
    case 64: return launch<64, G>(map_w, map_x, args, tiles, m_tiles, s);    \
    case 128: return launch<128, G>(map_w, map_x, args, tiles, m_tiles, s);  \
    case 256: return launch<256, G>(map_w, map_x, args, tiles, m_tiles, s);  \
    default: return -2;                                                      \
  }
  // the gated epilogue is a template instance of its own: the plain product then needs fewer
  // registers, and this kernel is measurably faster the fewer it holds
  if (gated) { BY_TILE(true) }
  BY_TILE(false)
#undef BY_TILE
}

int sb_gemm_tcgen05(const void* x, const void* w, void* out, int rows, int n_out, int k_dim, int bm,
                    int splits, int stages, int gated, int out_float, int* status, cudaStream_t s) {
  return gemm_entry(x, w, out, rows, n_out, k_dim, bm, splits, stages, gated, out_float, status,
                    WAIT_LIMIT_NS, -1, s);
}

// The same product with one activation copy left out on purpose (k-block `withhold_stage` of every
// CTA, which must be below `stages`) and waits that give up after `wait_limit_ns`: the kernel cannot
// finish the product and must return with bit 4 of *status set.  The output is then undefined.
int sb_gemm_tcgen05_withheld(const void* x, const void* w, void* out, int rows, int n_out, int k_dim, int bm,
                             int splits, int stages, int gated, int out_float, int* status,
                             unsigned long long wait_limit_ns, int withhold_stage, cudaStream_t s) {
  if (withhold_stage < 0 || withhold_stage >= stages || wait_limit_ns == 0) return -2;
  return gemm_entry(x, w, out, rows, n_out, k_dim, bm, splits, stages, gated, out_float, status,
                    wait_limit_ns, withhold_stage, s);
}

}  // extern "C"
