// y[m, n] = sum_k x[m, k] * w[n, k] in bfloat16 for MANY rows (prompts): a persistent kernel of CTA
// pairs on the fifth-generation tensor cores.
//
// Two CTAs (a cluster of two, on neighbouring SMs) own one [256 x BN] tile of y at a time: 256 rows of
// x (128 per CTA) against BN rows of w (BN / 2 per CTA).  Each CTA brings its own halves into its own
// shared memory by TMA ([128 x 64] and [BN / 2 x 64] boxes, 128-byte swizzle, K-major), every copy
// signalling the FIRST CTA's barrier of the stage (cp.async.bulk.tensor with .cta_group::2, no
// multicast).  One thread of the first CTA issues tcgen05.mma.cta_group::2 (M = 256, N = BN): the
// tensor cores of both SMs work on the same instruction, each reading its own x rows and both halves
// of w, and each CTA's tensor memory receives the 128 rows of the accumulator that belong to it.
// tcgen05.commit with cluster multicast hands the stage back to both CTAs' producers.
//
// The kernel is persistent: one CTA pair per pair of SMs, tiles dealt round robin in an order that
// keeps the tiles in flight close together (groups of row tiles, inside a group the row tiles of one
// weight tile next to each other), so that operands are read from memory once per group and from L2
// by the other tiles.  The accumulator is double buffered in tensor memory (2 x 256 columns): while the four
// epilogue warps of each CTA read tile i back (tcgen05.ld), round it and write it out, the tensor
// cores already work on tile i + 1.
//
// With `gated`, w is [gate; up] stacked ([2 * n_out, k]); the first CTA loads BN / 2 gate rows, the
// second the matching BN / 2 up rows, so a thread of the epilogue finds gate and up of the same output
// in its own accumulator row and writes round(silu(round(gate))) * round(up) (fused.py:89-112): the
// [rows, 2 * n_out] intermediate never exists.
//
// Every wait on an mbarrier gives up after a time limit, raises bit 4 of *status and lets both CTAs
// drain, free their tensor memory and return; sb_gemm_prompt_withheld leaves out one weight copy on
// purpose so that this path can be exercised without a fault.
#include "tcgen05.cuh"
#include "tensor_map.cuh"

#define PG_ROWS_PER_CTA 128
#define PG_TILE_M 256
#define PG_TILE_K 64
#define PG_A_BYTES (PG_ROWS_PER_CTA * PG_TILE_K * 2)
#define PG_THREADS 192
#define PG_MAX_STAGES 8
#define PG_ACC_STRIDE 256     // tensor-memory columns between the two accumulators
#define PG_TMEM_COLS 512

// ------------------------------------------------------------------------------------------ PTX

__device__ __forceinline__ uint32_t pg_cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// The address, in the cluster's shared window, of `addr` (an address of this CTA) in CTA `rank`.
__device__ __forceinline__ uint32_t pg_in_cta(uint32_t addr, uint32_t rank) {
  uint32_t a;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(a) : "r"(addr), "r"(rank));
  return a;
}
__device__ __forceinline__ void pg_cluster_sync() {
  asm volatile("barrier.cluster.arrive.release;\n\tbarrier.cluster.wait.acquire;" ::: "memory");
}
// One arrival on a barrier that may live in the other CTA of the pair (a shared::cluster address).
__device__ __forceinline__ void pg_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// A TMA tile load into this CTA's shared memory whose completion is counted on a barrier of either
// CTA of the pair (a shared::cluster address).
__device__ __forceinline__ void pg_tma_load(void* dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void pg_tmem_alloc(uint32_t* holder, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(holder)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void pg_tmem_free(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void pg_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// The barrier at this offset in BOTH CTAs gets one arrival when every MMA issued so far has completed.
__device__ __forceinline__ void pg_commit_both(uint64_t* bar) {
  const uint16_t both = 3;
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
               ::"r"(smem_u32(bar)), "h"(both) : "memory");
}
// 32 consecutive columns of this thread's accumulator row.
__device__ __forceinline__ void pg_tmem_load32(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// kind::f16: float accumulator, bfloat16 A and B, both K-major, M = 256 over the CTA pair, N = bn.
__device__ __forceinline__ uint32_t pg_instr_desc(int bn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(bn >> 3) << 17) | ((uint32_t)(PG_TILE_M >> 4) << 24);
}

struct PromptGemmArgs {
  bf16* out;            // [rows, n_out]
  const bf16* residual; // [rows, n_out] or null: out = round(residual + round(product)); may be `out` itself
  int* status;
  int rows, n_out, k_dim;
  int bn;               // weight rows per tile (the MMA's N); with gated, bn / 2 gate and bn / 2 up rows
  int stages, gated;
  int m_tiles, n_tiles;
  int group_m;          // row tiles per group (see pg_tile)
  unsigned long long wait_limit_ns;
  int withhold_kblock;  // >= 0: the first CTA leaves out its weight copy of this k-block of its first tile
};

// ------------------------------------------------------------------------------------------ kernel

// Which tile is the t-th.  Tiles that run at the same time (one per CTA pair, consecutive t) should
// share operands in L2: the row tiles are taken in groups of `group_m`; inside a group the tiles of
// one weight tile follow each other, then the next weight tile.  So at any time the pairs work on
// about group_m row tiles x a few weight tiles, the group's rows of x stay in L2 while all weight
// tiles pass, and the weights are read from memory once per group.
__device__ __forceinline__ void pg_tile(const PromptGemmArgs& args, int t, int& mt, int& nt) {
  const int per_group = args.group_m * args.n_tiles;
  const int g = t / per_group, r = t - g * per_group;
  const int here = min(args.group_m, args.m_tiles - g * args.group_m);
  nt = r / here;
  mt = g * args.group_m + (r - nt * here);
}

// 32 values of row `grow` starting at column `col` of out, rounded to bfloat16; with a residual
// stream, the rounded product is added to the stream's values first (the sum in float, rounded once
// more: what a separate add of two bfloat16 tensors gives, engine/engine.py:734-736).
__device__ __forceinline__ void pg_store32(const PromptGemmArgs& args, int grow, int col, float* v) {
  if (grow >= args.rows || col >= args.n_out) return;
  const size_t offset = (size_t)grow * args.n_out + col;
  bf16* at = args.out + offset;
  const bool wide = args.n_out % 8 == 0 && col + 32 <= args.n_out;
  if (args.residual) {
    const bf16* res = args.residual + offset;
    if (wide) {
#pragma unroll
      for (int j = 0; j < 32; j += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(res + j);
        const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
        for (int i = 0; i < 8; ++i) v[j + i] = __bfloat162float(e[i]) + rnd<bf16>(v[j + i]);
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j)
        if (col + j < args.n_out) v[j] = __bfloat162float(res[j]) + rnd<bf16>(v[j]);
    }
  }
  if (wide) {
#pragma unroll
    for (int j = 0; j < 32; j += 8) {
      __nv_bfloat162 p0 = __floats2bfloat162_rn(v[j], v[j + 1]), p1 = __floats2bfloat162_rn(v[j + 2], v[j + 3]);
      __nv_bfloat162 p2 = __floats2bfloat162_rn(v[j + 4], v[j + 5]), p3 = __floats2bfloat162_rn(v[j + 6], v[j + 7]);
      *reinterpret_cast<uint4*>(at + j) =
          make_uint4(*reinterpret_cast<uint32_t*>(&p0), *reinterpret_cast<uint32_t*>(&p1),
                     *reinterpret_cast<uint32_t*>(&p2), *reinterpret_cast<uint32_t*>(&p3));
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col + j < args.n_out) at[j] = __float2bfloat16_rn(v[j]);
  }
}

template <bool GATED>
__global__ void __launch_bounds__(PG_THREADS, 1)
gemm_prompt_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                   const PromptGemmArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  __shared__ uint64_t full_bar[PG_MAX_STAGES], empty_bar[PG_MAX_STAGES], acc_full[2], acc_empty[2], drain_bar;
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  const int STAGES = args.stages;
  const int half_n = args.bn / 2;                              // weight rows this CTA loads per tile
  const int B_BYTES = half_n * PG_TILE_K * 2;
  const int STAGE_BYTES = PG_A_BYTES + B_BYTES;
  const uint64_t limit = args.wait_limit_ns;
  // the warp's number as a value the compiler knows to be the same in every lane
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  const uint32_t rank = pg_cluster_rank();                     // 0: the CTA that issues the MMAs
  const int pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;
  const int n_tiles_total = args.m_tiles * args.n_tiles;
  const int n_kb = (args.k_dim + PG_TILE_K - 1) / PG_TILE_K;
  const int out_per_tile = GATED ? half_n : args.bn;           // output columns a tile covers

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 8); }
    mbar_init(&drain_bar, 1);
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 1) pg_tmem_alloc(&tmem_holder, PG_TMEM_COLS);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  pg_cluster_sync();     // both CTAs' barriers exist before either signals the other's
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  pdl_trigger();
  const uint32_t tmem = tmem_holder;
  volatile int* abort = &abort_flag;

  if (warp == 0) {
    // ---------------- producer: the warp walks the ring together, one elected lane issues the copies
    const bool elected = elect_one();
    pdl_wait();
    int it = 0, s = 0;
    uint32_t parity = 1;          // flips at every wrap of the ring; the first pass waits for nothing
    bool gave_up = false;
    for (int t = pair; t < n_tiles_total && !gave_up; t += n_pairs) {
      int mt, nt;
      pg_tile(args, t, mt, nt);
      const int m0 = mt * PG_TILE_M + (int)rank * PG_ROWS_PER_CTA;
      const int w0 = GATED ? (rank == 0 ? nt * half_n : args.n_out + nt * half_n) : nt * args.bn + (int)rank * half_n;
      const bool withheld_tile = rank == 0 && t == pair;
      for (int kb = 0; kb < n_kb; ++kb, ++it) {
        if (it >= STAGES && !__all_sync(0xffffffffu, mbar_wait(&empty_bar[s], parity, abort, limit))) { gave_up = true; break; }
        uint8_t* a = smem + (size_t)s * STAGE_BYTES;
        const uint32_t full = pg_in_cta(smem_u32(&full_bar[s]), 0);
        if (elected) {
          if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * STAGE_BYTES);
          pg_tma_load(a, &map_x, full, kb * PG_TILE_K, m0);
          if (!(withheld_tile && kb == args.withhold_kblock))
            pg_tma_load(a + PG_A_BYTES, &map_w, full, kb * PG_TILE_K, w0);
        }
        if (++s == STAGES) { s = 0; parity ^= 1; }
      }
    }
    if (*abort && elected) {
      // copies still in flight write into this CTA's shared memory: give them time to land
      const uint64_t start = now_ns();
      while (now_ns() - start < 100000ull) {}
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer: the warp of the first CTA walks the ring together (so that what
    // the MMAs take, descriptors and addresses, is the same in every lane and can live in the
    // uniform registers the instruction wants); one elected lane issues
    if (rank == 0) {
      const bool elected = elect_one();
      const uint32_t idesc = pg_instr_desc(args.bn);
      int it = 0, i = 0, s = 0;
      uint32_t parity = 0;
      bool gave_up = false;
      for (int t = pair; t < n_tiles_total && !gave_up; t += n_pairs, ++i) {
        const int b = i & 1;
        if (i >= 2 && !__all_sync(0xffffffffu, mbar_wait(&acc_empty[b], ((i >> 1) - 1) & 1, abort, limit))) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t d = tmem + (uint32_t)b * PG_ACC_STRIDE;
        for (int kb = 0; kb < n_kb; ++kb, ++it) {
          if (!__all_sync(0xffffffffu, mbar_wait(&full_bar[s], parity, abort, limit))) { gave_up = true; break; }
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t a_addr = smem_u32(smem + (size_t)s * STAGE_BYTES);
          const uint64_t a_desc = smem_desc(a_addr), b_desc = smem_desc(a_addr + PG_A_BYTES);
          if (elected) {
#pragma unroll
            for (int k = 0; k < PG_TILE_K / 16; ++k)
              pg_mma(d, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
            pg_commit_both(&empty_bar[s]);
          }
          __syncwarp();
          if (++s == STAGES) { s = 0; parity ^= 1; }
        }
        if (!gave_up && elected) pg_commit_both(&acc_full[b]);
        __syncwarp();
      }
      if (*abort && elected) {
        // the MMAs issued so far must be over before tensor memory and shared memory are given up
        asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                     ::"r"(smem_u32(&drain_bar)) : "memory");
        const uint64_t start = now_ns();
        while (!mbar_try(&drain_bar, 0) && now_ns() - start < limit) {}
      }
    }
  } else {
    // ---------------- epilogue: warps 2..5 own the tensor-memory lane quarters 2, 3, 0, 1
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const uint32_t lane_base = tmem + ((uint32_t)(quarter * 32) << 16);
    const uint32_t empty0 = pg_in_cta(smem_u32(&acc_empty[0]), 0), empty1 = pg_in_cta(smem_u32(&acc_empty[1]), 0);
    pdl_wait();   // before the first store: the output may be memory an earlier kernel still reads
    int i = 0;
    for (int t = pair; t < n_tiles_total; t += n_pairs, ++i) {
      const int b = i & 1;
      // the whole warp goes on or the whole warp stops: the reads below are warp-wide instructions
      if (!__all_sync(0xffffffffu, mbar_wait(&acc_full[b], (i >> 1) & 1, abort, limit))) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      int mt, nt;
      pg_tile(args, t, mt, nt);
      const int grow = mt * PG_TILE_M + (int)rank * PG_ROWS_PER_CTA + row;
      const int col0 = nt * out_per_tile;
      const uint32_t acc = lane_base + (uint32_t)b * PG_ACC_STRIDE;
      const int n_chunks = out_per_tile / 32;
#pragma unroll 1
      for (int c = 0; c < n_chunks; ++c) {
        float v[32];
        pg_tmem_load32(acc + c * 32, v);
        if (GATED) {
          float u[32];
          pg_tmem_load32(acc + half_n + c * 32, u);
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float gr = rnd<bf16>(v[j]), ur = rnd<bf16>(u[j]);
            v[j] = rnd<bf16>(gr / (1.f + __expf(-gr))) * ur;
          }
        }
        if (c == n_chunks - 1) {
          // this warp has read all it needs of the accumulator: the tensor cores may have it back
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          __syncwarp();
          if (lane == 0) pg_arrive_cluster(b ? empty1 : empty0);
        }
        pg_store32(args, grow, col0 + c * 32, v);
      }
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  pg_cluster_sync();     // nobody leaves while the other CTA may still signal its barriers or read its memory
  if (warp == 1) pg_tmem_free(tmem, PG_TMEM_COLS);
  if (threadIdx.x == 0 && abort_flag && args.status) atomicOr(args.status, 4);
}

// ------------------------------------------------------------------------------------------ host

static int pg_sm_count() {
  static int sms = 0;
  if (!sms) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  }
  return sms;
}

template <bool GATED>
static int pg_launch(const CUtensorMap& map_x, const CUtensorMap& map_w, const PromptGemmArgs& args, int pairs,
                     int smem, cudaStream_t s) {
  static int configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(gemm_prompt_kernel<GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  return launch_dependent_cluster(gemm_prompt_kernel<GATED>, dim3(2 * pairs), dim3(PG_THREADS), smem, s,
                                  dim3(2, 1, 1), map_x, map_w, args);
}

// x [rows, k_dim] and w [n_out (2 * n_out if gated), k_dim] bfloat16, row-major, 16-byte aligned, k_dim
// a multiple of 8; out [rows, n_out] bfloat16; residual null or [rows, n_out] bfloat16 (not with gated).  bn (0: chosen here) is the number of weight rows per
// tile: a multiple of 32 from 64 to 256 (of 64 if gated); pairs (0: one per two SMs) the number of CTA
// pairs.  Returns -2 for sizes it does not take, -3/-4 if the tensor maps cannot be made.
static int pg_entry(const void* x, const void* w, void* out, const void* residual, int rows, int n_out, int k_dim, int bn, int pairs,
                    int gated, int* status, unsigned long long wait_limit_ns, int withhold_kblock,
                    cudaStream_t s) {
  if (rows == 0 || n_out == 0) return 0;
  if (k_dim % 8 || k_dim <= 0) return -2;
  if (((uintptr_t)x | (uintptr_t)w) & 15) return -2;
  const int max_pairs = pg_sm_count() / 2;
  if (max_pairs < 1) return -2;
  if (pairs <= 0 || pairs > max_pairs) pairs = max_pairs;
  const int m_tiles = (rows + PG_TILE_M - 1) / PG_TILE_M;
  if (bn == 0) {
    // the least time on the busiest CTA pair: rounds of tiles times what a tile of that width takes
    // (measured: a k-block costs about 150 ns and 1.04 ns per weight row of the tile)
    long long best = -1;
    const int candidates[4] = {256, 192, 160, 128};
    for (int c = 0; c < 4; ++c) {
      const int cand = candidates[c];
      if (gated && cand % 64) continue;
      const int per = gated ? cand / 2 : cand;
      const long long tiles = (long long)m_tiles * ((n_out + per - 1) / per);
      const long long cost = ((tiles + pairs - 1) / pairs) * (cand + 144);
      if (best < 0 || cost < best) { best = cost; bn = cand; }
    }
  }
  if (bn < 64 || bn > 256 || bn % 32 || (gated && bn % 64)) return -2;
  const int per = gated ? bn / 2 : bn;
  const int n_tiles = (n_out + per - 1) / per;
  const int stage_bytes = PG_A_BYTES + (bn / 2) * PG_TILE_K * 2;
  int stages = (227 * 1024 - 1024 - 1024) / stage_bytes;
  if (stages > PG_MAX_STAGES) stages = PG_MAX_STAGES;
  if (stages < 2) return -2;
  const long long total = (long long)m_tiles * n_tiles;
  if (total < pairs) pairs = (int)total;
  CUtensorMap map_x, map_w;
  int rc = sb_make_map(&map_x, x, rows, k_dim, PG_ROWS_PER_CTA);
  if (rc) return rc;
  rc = sb_make_map(&map_w, w, gated ? 2ll * n_out : n_out, k_dim, bn / 2);
  if (rc) return rc;
  PromptGemmArgs args;
  if (residual && gated) return -2;
  args.out = (bf16*)out; args.residual = (const bf16*)residual; args.status = status;
  args.rows = rows; args.n_out = n_out; args.k_dim = k_dim;
  args.bn = bn; args.stages = stages; args.gated = gated;
  args.m_tiles = m_tiles; args.n_tiles = n_tiles;
  // a group's rows of x (group_m x 256 x k x 2 bytes) should stay in L2 beside the weights passing by
  long long group_m = (48ll << 20) / (512ll * k_dim);
  if (group_m > 16) group_m = 16;
  if (group_m < 1) group_m = 1;
  if (group_m > m_tiles) group_m = m_tiles;
  args.group_m = (int)group_m;
  args.wait_limit_ns = wait_limit_ns; args.withhold_kblock = withhold_kblock;
  const int smem = stages * stage_bytes + 1024;
  return gated ? pg_launch<true>(map_x, map_w, args, pairs, smem, s)
               : pg_launch<false>(map_x, map_w, args, pairs, smem, s);
}

extern "C" {

int sb_gemm_prompt(const void* x, const void* w, void* out, const void* residual, int rows, int n_out, int k_dim, int bn, int pairs,
                   int gated, int* status, cudaStream_t s) {
  return pg_entry(x, w, out, residual, rows, n_out, k_dim, bn, pairs, gated, status, TC_WAIT_LIMIT_NS, -1, s);
}

// The same product with one weight copy left out on purpose (k-block `withhold_kblock` of the first
// tile of every first CTA) and waits that give up after `wait_limit_ns`: the kernel cannot finish and
// must return with bit 4 of *status set.  The output is then undefined.
int sb_gemm_prompt_withheld(const void* x, const void* w, void* out, int rows, int n_out, int k_dim, int bn,
                            int pairs, int gated, int* status, unsigned long long wait_limit_ns,
                            int withhold_kblock, cudaStream_t s) {
  if (withhold_kblock < 0 || wait_limit_ns == 0) return -2;
  return pg_entry(x, w, out, nullptr, rows, n_out, k_dim, bn, pairs, gated, status, wait_limit_ns, withhold_kblock, s);
}

}  // extern "C"
