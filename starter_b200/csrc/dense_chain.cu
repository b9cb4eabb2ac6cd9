// A chain of few-row projections and row norms as ONE persistent kernel: for instance the output
// projection, the residual sum with the norm after it, the gated feed-forward's two projections, the
// next residual sum and norm and the next layer's q/k/v projection, which a decode step otherwise
// runs as six launches with a latency chain of several microseconds between each two.
//
// One CTA per SM stays resident for the whole chain.  Stages are of two kinds:
//   LINEAR  y[m, n] = sum_k x[m, k] * w[n, k] (bfloat16, float accumulation in tensor memory, the
//           weight's 128 rows as the MMA's M and up to 64 activation rows as its N, as in
//           gemm_tcgen05.cu), optionally gated (w = [gate; up], result round(silu(gate)) * up);
//   NORM    x = round(x + delta) written back, y = gain * round(x * rsqrt(mean(x^2) + eps))
//           (elementwise.cu's arithmetic, engine/kernels/fused.py:115-144), delta being either a
//           tensor given from outside or the LINEAR stage before it.
//
// How the work is cut: a LINEAR stage's (weight tile, k-block) pairs are numbered tile by tile and
// every CTA takes an equal, contiguous range of them, so every SM streams the same number of weight
// bytes whatever the shape.  A range that ends inside a tile leaves a partial tile; partial tiles go
// to a float scratch in global memory (it stays in L2) and are summed in the order of the CTAs that
// made them, so the sum does not depend on timing.  Who sums: for a LINEAR followed by a NORM, the
// CTA that norms a row sums that row's partials on the way; otherwise the CTAs take tiles in turn,
// sum, apply the gate if there is one, round and store.
//
// What keeps memory busy: a producer thread per CTA walks the WHOLE chain's weight tiles in order
// and keeps a ring of shared-memory slots full by TMA.  Weights depend on nothing, so it runs ahead
// of the stage that is computing, across stage boundaries, as far as the ring reaches (about
// 200 KB per SM, 29 MB over the chip: more than a whole small projection).  Activations are loaded
// by a second producer thread that waits for the stage before to be complete.
//
// Stages are separated by barriers over the whole grid: a counter in global memory that every CTA
// adds to and then polls.  All CTAs are resident at once (one per SM, the grid is never larger than
// the SM count), which is what makes waiting for each other legal.  Every wait (on an mbarrier, on
// the grid counter) gives up after a time limit, raises bit 32 of *status and a flag in the sync
// area that makes all other CTAs (and later launches, until the host clears it) give up at once.
#include "tcgen05.cuh"
#include "tensor_map.cuh"

#define DC_TILE_N 128
#define DC_TILE_K 64
#define DC_W_BYTES (DC_TILE_N * DC_TILE_K * 2)
#define DC_HALF_BYTES (64 * DC_TILE_K * 2)
#define DC_THREADS 256
#define DC_MAIN_THREADS 128          // warps 4..7: tensor-memory read-back, sums, norms, grid barriers
#define DC_MAX_STAGES 8
#define DC_MAX_LINEAR 6
#define DC_MAX_SLOTS 14
#define DC_KIND_LINEAR 0
#define DC_KIND_NORM 1
#define DC_STATUS_BIT 32

struct DcStage {
  int kind;
  // LINEAR
  int n_out;             // output features (of each half if gated)
  int k_dim;
  int gated;
  int store;             // 1: sum the partial tiles, finish and store to `out`; 0: a NORM stage follows and sums
  int parts_alloc;       // partial tiles kept per weight tile in `partial`
  void* out;             // [rows, n_out] bfloat16
  float* partial;        // [tiles][parts_alloc][bm][128] float
  // NORM
  int hidden;
  int gain_float;
  float eps;
  int has_residual;      // 0: the input is delta alone (nothing is added or written back)
  void* residual;        // [rows, hidden] bfloat16, read and written back
  const void* delta;     // [rows, hidden] bfloat16 from outside, or null: the LINEAR stage before
  const void* gain;
  void* normed;          // [rows, hidden] bfloat16
};

struct DcParams {
  DcStage st[DC_MAX_STAGES];
  int n_stages, rows, slots, norm_floats;
  unsigned long long* sync;      // [0] barrier counter, [1] abort flag
  int* status;
  unsigned long long limit_ns;
  unsigned long long* trace;     // null, or [ctas][64] time stamps (ns): 0.. main flow, 32.. weight producer, 48.. MMA
};

struct DcMaps {
  CUtensorMap w[DC_MAX_LINEAR];
  CUtensorMap x[DC_MAX_LINEAR];
};

// ------------------------------------------------------------------------------------------ helpers

__device__ __forceinline__ void named_sync(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
  unsigned long long v;
  asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void red_release_add_u64(unsigned long long* p, unsigned long long v) {
  asm volatile("red.release.gpu.global.add.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// Orders this thread's ordinary global accesses with the TMA unit's (the asynchronous proxy).
__device__ __forceinline__ void fence_async_global() { asm volatile("fence.proxy.async.global;" ::: "memory"); }

// The (tile, k-block) pairs of a LINEAR stage, numbered tile by tile, and who owns which.
struct DcCut {
  int kb_tile, tiles;
  long long total;
  int n_ctas;
  __device__ __forceinline__ void init(const DcStage& st, int ctas) {
    kb_tile = (st.k_dim + DC_TILE_K - 1) / DC_TILE_K;
    tiles = st.gated ? st.n_out / 64 : (st.n_out + DC_TILE_N - 1) / DC_TILE_N;
    total = (long long)tiles * kb_tile;
    n_ctas = ctas;
  }
  __device__ __forceinline__ long long begin_of(int cta) const { return (long long)cta * total / n_ctas; }
  // the CTA whose range holds pair g: the largest c with begin_of(c) <= g
  __device__ __forceinline__ int owner(long long g) const { return (int)(((g + 1) * n_ctas - 1) / total); }
  __device__ __forceinline__ int first_part(int tile) const { return owner((long long)tile * kb_tile); }
  __device__ __forceinline__ int parts(int tile) const {
    return owner((long long)(tile + 1) * kb_tile - 1) - first_part(tile) + 1;
  }
  // With fewer pairs than CTAs some CTAs between a tile's first and last owner own nothing; their
  // slot among the tile's partial tiles is never written and must not be read.
  __device__ __forceinline__ bool sparse() const { return total < n_ctas; }
  __device__ __forceinline__ bool owns_nothing(int c) const { return begin_of(c) == begin_of(c + 1); }
};

// A CTA's ranges within one stage, one per tile it touches.
struct DcSegments {
  long long at, end;
  int kb_tile;
  __device__ __forceinline__ void init(const DcCut& cut, int cta) {
    at = cut.begin_of(cta);
    end = cut.begin_of(cta + 1);
    kb_tile = cut.kb_tile;
  }
  __device__ __forceinline__ bool next(int& tile, int& k0, int& k1) {
    if (at >= end) return false;
    tile = (int)(at / kb_tile);
    k0 = (int)(at - (long long)tile * kb_tile);
    const long long left = end - at;
    k1 = (int)(left < (long long)(kb_tile - k0) ? k0 + left : kb_tile);
    at += k1 - k0;
    return true;
  }
};

template <int N> __device__ __forceinline__ void load_bf16x(const bf16* p, float* out) {
  if (N == 8) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const bf16* e = reinterpret_cast<const bf16*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = __bfloat162float(e[i]);
  }
}
__device__ __forceinline__ void store_bf16x8(bf16* p, const float* v) {
  uint4 raw;
  uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    __nv_bfloat162 two = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    w[i] = *reinterpret_cast<uint32_t*>(&two);
  }
  *reinterpret_cast<uint4*>(p) = raw;
}

// ------------------------------------------------------------------------------------------ kernel

struct DcShared {
  uint64_t full[DC_MAX_SLOTS], empty[DC_MAX_SLOTS], acc_full[2], acc_empty[2], ready;
  unsigned long long sync_base;
  uint32_t tmem;
  int abort;
  float red[8];
};

template <int BM>
__global__ void __launch_bounds__(DC_THREADS, 1)
dense_chain_kernel(const __grid_constant__ DcMaps maps, const __grid_constant__ DcParams p) {
  constexpr int X_BYTES = BM * DC_TILE_K * 2;
  constexpr int SLOT_BYTES = DC_W_BYTES + X_BYTES;
  constexpr uint32_t TMEM_COLS = 2 * BM < 32 ? 32 : 2 * BM;   // two accumulators in turn

  extern __shared__ uint8_t smem_raw[];
  uint8_t* ring = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* norm_buf = reinterpret_cast<float*>(ring + (size_t)p.slots * SLOT_BYTES);
  __shared__ DcShared sh;

  // the warp's number as a value the compiler knows to be the same in every lane
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;
  const int cta = blockIdx.x, n_ctas = gridDim.x;
  const int SLOTS = p.slots;
  const uint64_t limit = p.limit_ns;
  const int rows = p.rows;
  volatile int* abort = &sh.abort;

  if (threadIdx.x == 0) {
    for (int s = 0; s < SLOTS; ++s) { mbar_init(&sh.full[s], 2); mbar_init(&sh.empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&sh.acc_full[a], 1); mbar_init(&sh.acc_empty[a], 4); }
    mbar_init(&sh.ready, 1);
    sh.abort = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_trigger();
  if (warp == 2) tmem_alloc(&sh.tmem, TMEM_COLS);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = sh.tmem;

  if (warp == 0) {
    // ---------------- weight producer: runs ahead of everything, bounded by the ring alone.  The
    // whole warp walks the schedule and one elected lane issues the copies: addresses and coordinates
    // are then the same in every lane and can live in the uniform registers the copies want (run by
    // one lane inside a branch on the lane number, each copy or MMA costs over a hundred cycles to issue)
    {
      const bool elected = elect_one();
      int i = 0, lin = 0;
      for (int s = 0; s < p.n_stages && !*abort; ++s) {
        const DcStage& st = p.st[s];
        if (st.kind != DC_KIND_LINEAR) continue;
        DcCut cut; cut.init(st, n_ctas);
        DcSegments seg; seg.init(cut, cta);
        int tile, k0, k1;
        if (p.trace && elected) p.trace[(size_t)cta * 64 + 32 + 2 * lin] = now_ns();
        while (seg.next(tile, k0, k1)) {
          const int row_a = st.gated ? tile * 64 : tile * DC_TILE_N;
          const int row_b = st.gated ? st.n_out + tile * 64 : tile * DC_TILE_N + 64;
          for (int kb = k0; kb < k1; ++kb, ++i) {
            const int slot = i % SLOTS;
            if (i >= SLOTS && !__all_sync(0xffffffffu, mbar_wait(&sh.empty[slot], ((i / SLOTS) - 1) & 1, abort, limit))) break;
            uint8_t* dst = ring + (size_t)slot * SLOT_BYTES;
            if (elected) {
              mbar_expect_tx(&sh.full[slot], DC_W_BYTES);
              tma_load_2d(dst, &maps.w[lin], &sh.full[slot], kb * DC_TILE_K, row_a);
              tma_load_2d(dst + DC_HALF_BYTES, &maps.w[lin], &sh.full[slot], kb * DC_TILE_K, row_b);
            }
          }
          if (*abort) break;
        }
        if (p.trace && elected) p.trace[(size_t)cta * 64 + 32 + 2 * lin + 1] = now_ns();
        ++lin;
      }
    }
  } else if (warp == 1) {
    // ---------------- activation producer: a stage's input exists once the stage before is complete
    {
      const bool elected = elect_one();
      int i = 0, lin = 0;
      for (int s = 0; s < p.n_stages && !*abort; ++s) {
        const DcStage& st = p.st[s];
        if (st.kind != DC_KIND_LINEAR) continue;
        if (!__all_sync(0xffffffffu, mbar_wait(&sh.ready, lin & 1, abort, limit))) break;
        if (lin == 0) pdl_wait();
        fence_async_global();
        DcCut cut; cut.init(st, n_ctas);
        DcSegments seg; seg.init(cut, cta);
        int tile, k0, k1;
        while (seg.next(tile, k0, k1)) {
          for (int kb = k0; kb < k1; ++kb, ++i) {
            const int slot = i % SLOTS;
            if (i >= SLOTS && !__all_sync(0xffffffffu, mbar_wait(&sh.empty[slot], ((i / SLOTS) - 1) & 1, abort, limit))) break;
            if (elected) {
              mbar_expect_tx(&sh.full[slot], X_BYTES);
              tma_load_2d(ring + (size_t)slot * SLOT_BYTES + DC_W_BYTES, &maps.x[lin], &sh.full[slot],
                          kb * DC_TILE_K, 0);
            }
          }
          if (*abort) break;
        }
        ++lin;
      }
    }
  } else if (warp == 2) {
    // ---------------- MMA issuer: one accumulator per range, two accumulators in turn
    {
      const bool elected = elect_one();
      const uint32_t idesc = instr_desc(BM);
      int i = 0, use = 0, lin = 0;
      for (int s = 0; s < p.n_stages && !*abort; ++s) {
        const DcStage& st = p.st[s];
        if (st.kind != DC_KIND_LINEAR) continue;
        DcCut cut; cut.init(st, n_ctas);
        DcSegments seg; seg.init(cut, cta);
        int tile, k0, k1;
        while (seg.next(tile, k0, k1)) {
          const int a = use & 1;
          if (p.trace) {
            const bool first = elected && p.trace[(size_t)cta * 64 + 48 + 2 * lin] == 0;
            if (__any_sync(0xffffffffu, first)) {
              mbar_wait(&sh.full[i % SLOTS], (i / SLOTS) & 1, abort, limit);
              if (first) p.trace[(size_t)cta * 64 + 48 + 2 * lin] = now_ns();
            }
            __syncwarp();
          }
          if (use >= 2 && !__all_sync(0xffffffffu, mbar_wait(&sh.acc_empty[a], ((use >> 1) - 1) & 1, abort, limit))) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint32_t acc = tmem + (uint32_t)(a * BM);
          for (int kb = k0; kb < k1; ++kb, ++i) {
            const int slot = i % SLOTS;
            if (!__all_sync(0xffffffffu, mbar_wait(&sh.full[slot], (i / SLOTS) & 1, abort, limit))) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t a_addr = smem_u32(ring + (size_t)slot * SLOT_BYTES);
            const uint64_t a_desc = smem_desc(a_addr), b_desc = smem_desc(a_addr + DC_W_BYTES);
            if (elected) {
#pragma unroll
              for (int k = 0; k < DC_TILE_K / 16; ++k)
                umma_bf16(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > k0 || k > 0) ? 1u : 0u);
              umma_commit(&sh.empty[slot]);
            }
            __syncwarp();
          }
          if (__any_sync(0xffffffffu, *abort != 0)) break;
          if (elected) {
            umma_commit(&sh.acc_full[a]);
            if (p.trace) p.trace[(size_t)cta * 64 + 48 + 2 * lin + 1] = now_ns();
          }
          __syncwarp();
          ++use;
        }
        ++lin;
      }
    }
  } else if (warp >= 4) {
    // ---------------- main flow: read accumulators back, sum, norm, and keep the grid in step
    const int tid = threadIdx.x - 4 * 32;              // 0..127
    const int quarter = warp & 3;                      // the tensor-memory lanes this warp may read
    const int r = quarter * 32 + lane;                 // row of the weight tile
    const int rows_pad = (rows + 7) & ~7;

    pdl_wait();
    if (tid == 0) {
      const unsigned long long seen = ld_acquire_u64(p.sync);
      sh.sync_base = seen - seen % (unsigned long long)n_ctas;
      if (ld_relaxed_u64(p.sync + 1) != 0) sh.abort = 1;   // an earlier launch gave up: the counter is off
    }
    named_sync(1, DC_MAIN_THREADS);
    unsigned long long target = sh.sync_base;
    int stamps = 0;
    auto stamp = [&]() {
      if (p.trace && tid == 0 && stamps < 32) p.trace[(size_t)cta * 64 + stamps] = now_ns();
      ++stamps;
    };
    stamp();

    // One barrier over all CTAs.  False if it ran out of time (or another CTA said so).
    auto grid_barrier = [&]() -> bool {
      __threadfence();
      fence_async_global();
      named_sync(1, DC_MAIN_THREADS);
      target += (unsigned long long)n_ctas;
      if (tid == 0 && !*abort) {
        red_release_add_u64(p.sync, 1ull);
        const uint64_t start = now_ns();
#pragma unroll 1
        for (uint32_t spin = 0;; ++spin) {
          if (ld_acquire_u64(p.sync) >= target) break;
          if ((spin & 15) == 15) {
            if (ld_relaxed_u64(p.sync + 1) != 0 || now_ns() - start > limit) { *abort = 1; break; }
          }
        }
        __threadfence();
      }
      named_sync(1, DC_MAIN_THREADS);
      return !*abort;
    };

    // Row `row` of a NORM stage: the sum with its delta (from outside, or the partial tiles of the
    // LINEAR stage `lin_st`), written back, and its norm.
    auto norm_row = [&](const DcStage& st, const DcStage* lin_st, int row) {
      const int hidden = st.hidden;
      bf16* res = (bf16*)st.residual + (size_t)row * hidden;
      const bf16* ext = (const bf16*)st.delta;
      DcCut cut;
      if (lin_st) cut.init(*lin_st, n_ctas);
      float ss = 0.f;
      for (int c = tid * 8; c < hidden; c += DC_MAIN_THREADS * 8) {
        float d[8];
        if (lin_st) {
          const int tile = c / DC_TILE_N, col = c % DC_TILE_N;
          const int n_parts = cut.parts(tile), first = cut.first_part(tile);
          const float* src = lin_st->partial + (((size_t)tile * lin_st->parts_alloc) * BM + row) * DC_TILE_N + col;
#pragma unroll
          for (int j = 0; j < 8; ++j) d[j] = 0.f;
          // the loads of four parts are in flight together; the sums stay in part order
          for (int part = 0; part < n_parts; part += 4, src += (size_t)4 * BM * DC_TILE_N) {
            float4 lo[4], hi[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const bool live = part + q < n_parts && !(cut.sparse() && cut.owns_nothing(first + part + q));
              const float* at = src + (size_t)q * BM * DC_TILE_N;
              lo[q] = live ? __ldcg(reinterpret_cast<const float4*>(at)) : make_float4(0.f, 0.f, 0.f, 0.f);
              hi[q] = live ? __ldcg(reinterpret_cast<const float4*>(at + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              d[0] += lo[q].x; d[1] += lo[q].y; d[2] += lo[q].z; d[3] += lo[q].w;
              d[4] += hi[q].x; d[5] += hi[q].y; d[6] += hi[q].z; d[7] += hi[q].w;
            }
          }
#pragma unroll
          for (int j = 0; j < 8; j += 2) rnd2<bf16>(d[j], d[j + 1]);     // the projection's own rounding
        } else if (ext) {
          load_bf16x<8>(ext + (size_t)row * hidden + c, d);
        }
        float v[8];
        if (st.has_residual) {
          load_bf16x<8>(res + c, v);
          if (lin_st || ext) {
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
              v[j] += d[j];
              v[j + 1] += d[j + 1];
              rnd2<bf16>(v[j], v[j + 1]);
            }
            uint4 raw;
            uint32_t* w = reinterpret_cast<uint32_t*>(&raw);
#pragma unroll
            for (int j = 0; j < 4; ++j) w[j] = pack_exact_bf16(v[2 * j], v[2 * j + 1]);
            *reinterpret_cast<uint4*>(res + c) = raw;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) v[j] = d[j];
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          ss += v[j] * v[j];
          norm_buf[c + j] = v[j];
        }
      }
      ss = warp_sum(ss);
      if (lane == 0) sh.red[quarter] = ss;
      named_sync(1, DC_MAIN_THREADS);
      ss = sh.red[0] + sh.red[1] + sh.red[2] + sh.red[3];
      const float inv = rsqrtf(ss / (float)hidden + st.eps);
      bf16* out = (bf16*)st.normed + (size_t)row * hidden;
      for (int c = tid * 8; c < hidden; c += DC_MAIN_THREADS * 8) {
        float g[8], o[8];
        if (st.gain_float) {
          const float4 lo = *reinterpret_cast<const float4*>((const float*)st.gain + c);
          const float4 hi = *reinterpret_cast<const float4*>((const float*)st.gain + c + 4);
          g[0] = lo.x; g[1] = lo.y; g[2] = lo.z; g[3] = lo.w; g[4] = hi.x; g[5] = hi.y; g[6] = hi.z; g[7] = hi.w;
        } else {
          load_bf16x<8>((const bf16*)st.gain + c, g);
        }
#pragma unroll
        for (int j = 0; j < 8; j += 2) {
          float a = norm_buf[c + j] * inv, b = norm_buf[c + j + 1] * inv;
          rnd2<bf16>(a, b);
          o[j] = a * g[j];
          o[j + 1] = b * g[j + 1];
        }
        store_bf16x8(out + c, o);
      }
      named_sync(1, DC_MAIN_THREADS);      // norm_buf and sh.red are free again
    };

    // The partial tiles of a LINEAR stage with store = 1, summed, finished and stored; tiles in turn.
    auto store_tiles = [&](const DcStage& st) {
      DcCut cut; cut.init(st, n_ctas);
      const int cols = st.gated ? 64 : DC_TILE_N;
      const int per_row = cols / 4;
      const bool vec = st.n_out % 4 == 0;
      for (int tile = cta; tile < cut.tiles; tile += n_ctas) {
        const int n_parts = cut.parts(tile), first = cut.first_part(tile);
        const float* base = st.partial + ((size_t)tile * st.parts_alloc) * BM * DC_TILE_N;
        for (int item = tid; item < per_row * rows; item += DC_MAIN_THREADS) {
          const int m = item / per_row, col = (item - m * per_row) * 4;
          const float* src = base + (size_t)m * DC_TILE_N + col;
          float g[4] = {0.f, 0.f, 0.f, 0.f}, u[4] = {0.f, 0.f, 0.f, 0.f};
          for (int part = 0; part < n_parts; ++part, src += (size_t)BM * DC_TILE_N) {
            if (cut.sparse() && cut.owns_nothing(first + part)) continue;
            const float4 gv = __ldcg(reinterpret_cast<const float4*>(src));
            g[0] += gv.x; g[1] += gv.y; g[2] += gv.z; g[3] += gv.w;
            if (st.gated) {
              const float4 uv = __ldcg(reinterpret_cast<const float4*>(src + 64));
              u[0] += uv.x; u[1] += uv.y; u[2] += uv.z; u[3] += uv.w;
            }
          }
          if (st.gated) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const float gr = rnd<bf16>(g[j]), ur = rnd<bf16>(u[j]);
              g[j] = rnd<bf16>(gr / (1.f + __expf(-gr))) * ur;
            }
          }
          const int ncol = tile * cols + col;
          bf16* dst = (bf16*)st.out + (size_t)m * st.n_out + ncol;
          if (vec && ncol + 3 < st.n_out) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(g[0], g[1]), hi = __floats2bfloat162_rn(g[2], g[3]);
            *reinterpret_cast<uint2*>(dst) = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
          } else {
#pragma unroll
            for (int j = 0; j < 4; ++j)
              if (ncol + j < st.n_out) dst[j] = __float2bfloat16_rn(g[j]);
          }
        }
      }
    };

    int use = 0, lin = 0;
    bool alive = !*abort;
    for (int s = 0; s < p.n_stages && alive; ++s) {
      const DcStage& st = p.st[s];
      if (st.kind == DC_KIND_NORM) {
        // a norm whose delta comes from outside (one after a LINEAR stage is done further down)
        for (int row = cta; row < rows; row += n_ctas) norm_row(st, nullptr, row);
        if (s + 1 < p.n_stages) alive = grid_barrier();
        continue;
      }
      if (tid == 0) mbar_arrive(&sh.ready);            // this stage's input is complete: load it
      DcCut cut; cut.init(st, n_ctas);
      DcSegments seg; seg.init(cut, cta);
      int tile, k0, k1;
      while (alive && seg.next(tile, k0, k1)) {
        const int a = use & 1;
        if (!mbar_wait(&sh.acc_full[a], (use >> 1) & 1, abort, limit)) { alive = false; break; }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const int part = cta - cut.first_part(tile);
        float* dst = st.partial + (((size_t)tile * st.parts_alloc + part) * BM) * DC_TILE_N + r;
#pragma unroll 1
        for (int c = 0; c < rows_pad; c += 8) {
          float v[8];
          tmem_load8(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(a * BM + c), v);
#pragma unroll
          for (int j = 0; j < 8; ++j)
            if (c + j < rows) dst[(size_t)(c + j) * DC_TILE_N] = v[j];
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&sh.acc_empty[a]);
        ++use;
      }
      ++lin;
      if (!alive) break;
      stamp();
      alive = grid_barrier();                          // every CTA's partial tiles are in place
      if (!alive) break;
      stamp();
      if (st.store) {
        store_tiles(st);
      } else {
        const DcStage& norm = p.st[s + 1];
        for (int row = cta; row < rows; row += n_ctas) norm_row(norm, &st, row);
        ++s;
      }
      stamp();
      if (s + 1 < p.n_stages) alive = grid_barrier();  // the stage's result is complete
      stamp();
    }
    if (*abort && tid == 0) {
      atomicExch(p.sync + 1, 1ull);                    // everyone else, and later launches, give up too
      // copies that are still on their way write into this CTA's shared memory: give them time
      const uint64_t start = now_ns();
      while (now_ns() - start < 50000ull) {}
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 2) tmem_free(tmem, TMEM_COLS);
  if (threadIdx.x == 0 && sh.abort && p.status) atomicOr(p.status, DC_STATUS_BIT);
}

// ------------------------------------------------------------------------------------------ host

static int dc_sm_count() {
  static int count[64];
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 0;
  if (!count[device]) cudaDeviceGetAttribute(&count[device], cudaDevAttrMultiProcessorCount, device);
  return count[device];
}

template <int BM>
static int dc_launch(const DcMaps& maps, DcParams& params, int grid, cudaStream_t s) {
  constexpr int SLOT_BYTES = DC_W_BYTES + BM * DC_TILE_K * 2;
  const int norm_bytes = params.norm_floats * 4;
  int slots = (225 * 1024 - 1024 - norm_bytes) / SLOT_BYTES;   // 227 KB per CTA, less the static part
  if (slots > DC_MAX_SLOTS) slots = DC_MAX_SLOTS;
  if (slots < 2) return -2;
  params.slots = slots;
  const int smem = slots * SLOT_BYTES + norm_bytes + 1024;
  static int configured = 0;
  if (smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(dense_chain_kernel<BM>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = smem;
  }
  return launch_dependent(dense_chain_kernel<BM>, dim3(grid), dim3(DC_THREADS), smem, s, maps, params);
}

extern "C" {

// How many CTAs a chain runs as on the current device (one per SM): the partial-tile scratch of a
// LINEAR stage is sized from it (see sb_dense_chain_parts).
int sb_dense_chain_ctas(void) { return dc_sm_count(); }

// The most partial tiles any weight tile of a LINEAR stage gets when `n_ctas` CTAs share its
// (tile, k-block) pairs: the second dimension of the stage's scratch [tiles][parts][bm][128].
int sb_dense_chain_parts(int n_out, int k_dim, int gated, int n_ctas) {
  const int kb_tile = (k_dim + DC_TILE_K - 1) / DC_TILE_K;
  const int tiles = gated ? n_out / 64 : (n_out + DC_TILE_N - 1) / DC_TILE_N;
  const long long total = (long long)tiles * kb_tile;
  if (total <= 0 || n_ctas <= 0) return 0;
  int most = 1;
  for (int tile = 0; tile < tiles; ++tile) {
    const int first = (int)((((long long)tile * kb_tile + 1) * n_ctas - 1) / total);
    const int last = (int)((((long long)(tile + 1) * kb_tile) * n_ctas - 1) / total);
    if (last - first + 1 > most) most = last - first + 1;
  }
  return most;
}

// One chain.  Per stage, 16 integers in `desc` (pointers as integers) and one float in `eps`:
//   [0] kind (0 LINEAR, 1 NORM)
//   LINEAR: [1] n_out [2] k_dim [3] gated [4] store [5] x [6] w [7] out [8] partial [9] parts_alloc
//   NORM:   [1] hidden [2] gain_float [3] has_residual [4] residual [5] delta (0: the LINEAR before
//           it if that has store = 0, else the residual alone is normed)
//           [6] gain [7] normed
// x of a LINEAR stage is [rows, k_dim] bfloat16; w is [n_out (2 * n_out if gated), k_dim]; all
// 16-byte aligned, k_dim and hidden multiples of 8, gated n_out a multiple of 64.  `sync` is two
// 64-bit words that start at zero and belong to the chains of one device (counter, abort flag).
// `trace` is null or room for 64 zeroed time stamps per CTA (see the kernel's stamp()).
// rows <= 64.  Returns -2 for what it does not take, -3/-4 if tensor maps cannot be made.
int sb_dense_chain(const long long* desc, const float* eps, int n_stages, int rows, unsigned long long* sync,
                   int* status, unsigned long long limit_ns, unsigned long long* trace, cudaStream_t s) {
  if (n_stages < 1 || n_stages > DC_MAX_STAGES || rows < 1 || rows > 64 || !sync) return -2;
  const int bm = rows <= 16 ? 16 : rows <= 32 ? 32 : 64;
  const int grid = dc_sm_count();
  if (grid <= 0) return -2;
  DcMaps maps;
  DcParams params;
  params.n_stages = n_stages;
  params.rows = rows;
  params.sync = sync;
  params.status = status;
  params.limit_ns = limit_ns ? limit_ns : TC_WAIT_LIMIT_NS;
  params.norm_floats = 0;
  params.trace = trace;
  int lin = 0;
  for (int i = 0; i < n_stages; ++i) {
    const long long* d = desc + 16 * i;
    DcStage& st = params.st[i];
    st = DcStage();
    st.kind = (int)d[0];
    if (st.kind == DC_KIND_LINEAR) {
      if (lin >= DC_MAX_LINEAR) return -2;
      st.n_out = (int)d[1]; st.k_dim = (int)d[2]; st.gated = (int)d[3]; st.store = (int)d[4];
      const void* x = (const void*)d[5];
      const void* w = (const void*)d[6];
      st.out = (void*)d[7]; st.partial = (float*)d[8]; st.parts_alloc = (int)d[9];
      if (st.n_out <= 0 || st.k_dim <= 0 || st.k_dim % 8 || (st.gated && st.n_out % 64)) return -2;
      if ((((uintptr_t)x | (uintptr_t)w | (uintptr_t)st.partial) & 15) || !st.partial) return -2;
      if (st.parts_alloc < sb_dense_chain_parts(st.n_out, st.k_dim, st.gated, grid)) return -2;
      if (st.store) {
        if (!st.out || ((uintptr_t)st.out & 7)) return -2;
      } else {
        // the NORM stage after it sums the tiles: it must be there and be as wide as this output
        if (i + 1 >= n_stages || (int)desc[16 * (i + 1)] != DC_KIND_NORM || desc[16 * (i + 1) + 5] != 0 ||
            (int)desc[16 * (i + 1) + 1] != st.n_out || st.gated)
          return -2;
      }
      int rc = sb_make_map(&maps.w[lin], w, st.gated ? 2ll * st.n_out : st.n_out, st.k_dim, 64);
      if (rc) return rc;
      rc = sb_make_map(&maps.x[lin], x, rows, st.k_dim, bm);
      if (rc) return rc;
      ++lin;
    } else if (st.kind == DC_KIND_NORM) {
      st.hidden = (int)d[1]; st.gain_float = (int)d[2]; st.has_residual = (int)d[3];
      st.residual = (void*)d[4]; st.delta = (const void*)d[5]; st.gain = (const void*)d[6];
      st.normed = (void*)d[7]; st.eps = eps[i];
      if (st.hidden <= 0 || st.hidden % 8 || !st.gain || !st.normed) return -2;
      if (st.has_residual && !st.residual) return -2;
      if ((((uintptr_t)st.residual | (uintptr_t)st.delta | (uintptr_t)st.gain | (uintptr_t)st.normed) & 15)) return -2;
      const bool after_open_linear = i > 0 && (int)desc[16 * (i - 1)] == DC_KIND_LINEAR && desc[16 * (i - 1) + 4] == 0;
      if (after_open_linear && st.delta) return -2;          // that stage's sum is this norm's delta
      if (!st.delta && !after_open_linear && !st.has_residual) return -2;   // nothing to norm
      if (st.hidden > params.norm_floats) params.norm_floats = st.hidden;
    } else {
      return -2;
    }
  }
  if (params.norm_floats * 4 > 64 * 1024) return -2;
  switch (bm) {
    case 16: return dc_launch<16>(maps, params, grid, s);
    case 32: return dc_launch<32>(maps, params, grid, s);
    default: return dc_launch<64>(maps, params, grid, s);
  }
}

}  // extern "C"
