// Causal grouped-query attention for prompts on the fifth-generation tensor cores (bfloat16).
//
// A block takes 256 consecutive query tokens of one sequence and one query head as two tiles of 128.
// Both products of a tile run as tcgen05.mma with the accumulators in tensor memory:
//     S  = Q K^T     M = 128 queries, N = 128 keys,  K = head_dim   (Q and K K-major)
//     O += P V       M = 128 queries, N = head_dim,  K = 128 keys   (V as it lies in the cache:
//                                                                    keys x head_dim, "MN-major")
// Tensor memory holds S of both tiles (2 x 128 columns) and O of both tiles (2 x 128 columns).
//
// Warps:   0-3 softmax of tile 0, 4-7 softmax of tile 1 (thread = query row = TMEM lane, so the
//          online softmax needs no shuffle: engine/kernels/fused.py:288-312),
//          8 TMA producer, 9 and 10 the MMA issuers of tile 0 and tile 1.
// TMA brings both Q tiles once and, per step of 128 keys (two cache pages), K and V with the
// 128-byte swizzle the tensor core reads; the keys alternate between two buffers and run a step
// ahead of the values, which have one buffer, because S of step i+1 is issued as soon as the softmax
// warps have read S of step i out of tensor memory, while PV of step i has to wait for P.
// The softmax warps write P = exp2(S * scale - m), rounded to bfloat16 (fused.py:699-701), into
// shared memory as the A operand of PV.  O stays in tensor memory and is accumulated by the MMA
// itself: m is the reference of the step before as long as no row's maximum outgrows it by more
// than 2^8 (P stays far inside bfloat16's range, the sum is kept in float); only then is O read,
// rescaled and written back, and the step's P redone.  The result is O / l, as in the exact online
// softmax, up to rounding.
// Keys are read from the cache like in every other attention kernel of this library, so a chunk
// that continues a sequence needs nothing special: a query at absolute position p sees keys j <= p
// (engine/engine.py:781-787) and, with a window w, j > p - w.
//
// Every wait on an mbarrier gives up after WAIT_LIMIT_NS, raises bit 16 of *status and lets the
// block drain its copies, free its tensor memory and return.
#include <cuda.h>

#include "common.cuh"
#include "tensor_map.cuh"

#define TC_BQ 128
#define TC_BK 128
#define TC_THREADS 352
#define TC_RING 3
#define WAIT_LIMIT_NS 2000000000ull

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// True in exactly one lane of the (converged) warp.
__device__ __forceinline__ bool elect_one() {
  uint32_t chosen;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(chosen));
  return chosen != 0;
}
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
// For tests of the give-up path (sb_attention_prefill_tc_withhold): how long a wait may take, and
// which step's values the producer leaves out (-1: none).  Read only once a wait has spun a while.
__device__ unsigned long long tc_wait_limit_ns = WAIT_LIMIT_NS;
__device__ int tc_withhold_step = -1;

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort) {
#pragma unroll 1
  for (int spin = 0; spin < 2048; ++spin)
    if (mbar_try(bar, parity)) return true;
  const uint64_t start = now_ns();
  const uint64_t limit = *(volatile unsigned long long*)&tc_wait_limit_ns;
#pragma unroll 1
  for (uint32_t spin = 0;; ++spin) {
    if (mbar_try(bar, parity)) return true;
    if ((spin & 63) == 0) {
      if (*abort) return false;
      if (now_ns() - start > limit) { *abort = 1; return false; }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc(uint32_t* holder, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(holder)), "r"(cols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t addr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(addr), "r"(cols) : "memory");
}
__device__ __forceinline__ void umma_bf16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 consecutive float columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_load32(uint32_t taddr, float* v) {
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

// 64 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_load64(uint32_t taddr, float* v) {
  uint32_t r[64];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
      "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
      "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];\n\t"
      "tcgen05.wait::ld.sync.aligned;"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
        "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
        "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
        "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
        "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
      : "r"(taddr)
      : "memory");
#pragma unroll
  for (int i = 0; i < 64; ++i) v[i] = __uint_as_float(r[i]);
}
// 32 columns back into this thread's TMEM lane
__device__ __forceinline__ void tmem_store32(uint32_t taddr, const float* v) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
        "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])), "r"(__float_as_uint(v[8])),
        "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])),
        "r"(__float_as_uint(v[15])), "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])),
        "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])), "r"(__float_as_uint(v[20])),
        "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])),
        "r"(__float_as_uint(v[27])), "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])),
        "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
// Two fused multiply-adds / two adds in one instruction (packed f32x2): half the issue slots.
__device__ __forceinline__ void fma2(float& d0, float& d1, float a0, float a1, float b, float c) {
  asm("{\n\t.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %4};\n\tmov.b64 rc, {%5, %5};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\tmov.b64 {%0, %1}, rd;\n\t}"
      : "=f"(d0), "=f"(d1) : "f"(a0), "f"(a1), "f"(b), "f"(c));
}
__device__ __forceinline__ void add2(float& acc0, float& acc1, float a0, float a1) {
  asm("{\n\t.reg .b64 ra, rb;\n\t"
      "mov.b64 ra, {%0, %1};\n\tmov.b64 rb, {%2, %3};\n\t"
      "add.rn.f32x2 ra, ra, rb;\n\tmov.b64 {%0, %1}, ra;\n\t}"
      : "+f"(acc0), "+f"(acc1) : "f"(a0), "f"(a1));
}
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Operand tile with rows of 128 bytes and 128-byte swizzle, 8-row groups 1024 bytes apart.  For a
// K-major operand the rows are M/N and `lbo` is unused; for an MN-major operand the rows are k and
// `lbo` is the distance between 64-element chunks along M/N.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((addr & 0x3FFFF) >> 4);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}
// kind::f16, float accumulator, bfloat16 operands, A K-major, M = 128; B K-major or MN-major.
__device__ __forceinline__ uint32_t instr_desc(int n, int b_mn_major) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)b_mn_major << 16) | ((uint32_t)(n >> 3) << 17) |
         ((uint32_t)(TC_BQ >> 4) << 24);
}

template <int D>
__global__ void __launch_bounds__(TC_THREADS, 1)
attention_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                            const __grid_constant__ CUtensorMap map_v, bf16* __restrict__ out,
                            const int* __restrict__ block_table, int table_stride,
                            const int* __restrict__ seq_slot, const int* __restrict__ seq_q_start,
                            const int* __restrict__ seq_q_len, const int* __restrict__ seq_kv_len,
                            const int* __restrict__ tile_seq, const int* __restrict__ tile_first,
                            int heads, int kv_heads, float scale_log2, int window, int* status, int list_of_blocks) {
  constexpr int DC = D / 64;                        // 64-element (128-byte) chunks of the head
  constexpr int SUB = 128 * 128;                    // bytes of a [128 rows x 128 bytes] sub-tile
  constexpr int Q_BYTES = DC * SUB;                 // one tile of 128 queries
  constexpr int KV_BYTES = DC * SUB;                // keys (or values) of 128 tokens
  constexpr int P_BYTES = 2 * SUB;                  // [128 queries x 128 keys] bfloat16
  constexpr uint32_t TMEM_COLS = 512;               // S of both tiles: 2 x 128; O of both tiles: 2 x 128
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* q_sm = smem;                             // 2 tiles
  uint8_t* p_sm = q_sm + 2 * Q_BYTES;               // 2 tiles
  uint8_t* ring = p_sm + 2 * P_BYTES;               // buffers 0 and 1: keys of even and odd steps; 2: values
  __shared__ uint64_t q_full, full[TC_RING], empty[TC_RING], s_ready[2], s_free[2], p_ready[2], o_ready[2];
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_flag;

  const int tile = blockIdx.y, head = blockIdx.x;   // heads run fastest: the work list's order holds
  const int q_first = tile_first[tile];
  // the work list is either this kernel's own (one entry per block of 256 queries) or the common
  // one in tiles of 64 queries, of which every fourth starts a block
  if (!list_of_blocks && (q_first & 255)) return;
  const int seq = tile_seq[tile];
  const int q_len = seq_q_len[seq], kv_len = seq_kv_len[seq];
  const int rows_valid = min(2 * TC_BQ, q_len - q_first);
  const int pos0 = kv_len - q_len + q_first;
  const int kvh = head / (heads / kv_heads);
  const int* pages = block_table + (size_t)seq_slot[seq] * table_stride;
  // the warp's number as a value the compiler knows to be the same in every lane
  const int warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = threadIdx.x & 31;

  const int hi = pos0 + rows_valid - 1;
  int lo = 0;
  if (window > 0 && pos0 - window + 1 > 0) lo = pos0 - window + 1;
  const int page_lo = lo / SB_PAGE_TOKENS, page_hi = hi / SB_PAGE_TOKENS;
  // steps of two pages (128 keys) that each tile of 128 queries needs, counted from page_lo
  int n_tile[2];
  n_tile[0] = ((pos0 + min(rows_valid, TC_BQ) - 1) / SB_PAGE_TOKENS - page_lo) / 2 + 1;
  n_tile[1] = rows_valid > TC_BQ ? (page_hi - page_lo) / 2 + 1 : 0;
  const int n_steps = max(n_tile[0], n_tile[1]);

  if (threadIdx.x == 0) {
    mbar_init(&q_full, 1);
    for (int s = 0; s < TC_RING; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 2); }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_ready[t], 1);
      mbar_init(&s_free[t], 4);       // one arrival per softmax warp
      mbar_init(&p_ready[t], 4);
      mbar_init(&o_ready[t], 1);
    }
    abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_trigger();
  if (warp == 9) tmem_alloc(&tmem_holder, TMEM_COLS);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_holder;
  volatile int* abort = &abort_flag;

  if (warp == 8) {
    // ---------------- producer: the whole warp walks the schedule, one elected lane issues the
    // copies (addresses and coordinates are then the same in every lane and can live in the uniform
    // registers the copy instructions want; run by one lane inside a branch on the lane number, each
    // copy costs over a hundred cycles to issue)
    {
      const bool elected = elect_one();
      pdl_wait();
      const int q_row0 = seq_q_start[seq] + q_first;
      const int q_tiles = n_tile[1] ? 2 : 1;
      if (elected) mbar_expect_tx(&q_full, q_tiles * Q_BYTES);
      for (int t = 0; t < q_tiles; ++t)
        for (int c = 0; c < DC; ++c)
          if (elected) tma_load_2d(q_sm + t * Q_BYTES + c * SUB, &map_q, &q_full, head * D + c * 64, q_row0 + t * TC_BQ);
      // Keys alternate between buffers 0 and 1 and run a step ahead of the values, which have
      // buffer 2: K0 V0 K1 | K2 V1 | K3 V2 ...  (S of step i+1 is issued early in step i, PV late.)
      auto load = [&](bool is_v, int i) -> bool {
        const int b = is_v ? 2 : (i & 1), use = is_v ? i : (i >> 1);
        if (use > 0 && !__all_sync(0xffffffffu, mbar_wait(&empty[b], (use - 1) & 1, abort))) return false;
        if (elected) mbar_expect_tx(&full[b], KV_BYTES);
        const bool withheld = is_v && i == *(volatile int*)&tc_withhold_step;   // tests only
        for (int half = 0; half < (withheld ? 1 : 2); ++half) {
          const int page = pages[min(page_lo + 2 * i + half, page_hi)];
          const int row = (page * kv_heads + kvh) * SB_PAGE_TOKENS;
          for (int c = 0; c < DC; ++c)
            if (elected) tma_load_2d(ring + b * KV_BYTES + c * SUB + half * 8192, is_v ? &map_v : &map_k, &full[b], c * 64, row);
        }
        return true;
      };
      int loads[3] = {0, 0, 0};                        // per buffer: how many copies were started
      bool ok = load(false, 0);
      if (ok) { loads[0]++; ok = load(true, 0); }
      if (ok) loads[2]++;
      if (ok && n_steps > 1) { ok = load(false, 1); if (ok) loads[1]++; }
      for (int i = 1; i < n_steps && ok; ++i) {
        if (i + 1 < n_steps) { ok = load(false, i + 1); if (ok) loads[(i + 1) & 1]++; }
        if (ok) { ok = load(true, i); if (ok) loads[2]++; }
      }
      if (*abort && elected) {                         // let the copies in flight land before the block ends
        for (int b = 0; b < 3; ++b) {
          const uint64_t start = now_ns();
          while (loads[b] > 0 && !mbar_try(&full[b], (loads[b] - 1) & 1) && now_ns() - start < WAIT_LIMIT_NS) {}
        }
      }
    }
  } else if (warp == 9 || warp == 10) {
    // ---------------- MMA issuers: warp 9 for tile 0, warp 10 for tile 1.  Each runs its own chain
    // of waits, so that one tile's waiting does not hold up the other's products.
    const int t = warp - 9, n_mine = n_tile[t], n_other = n_tile[1 - t];
    if (n_mine > 0) {
      // the whole warp waits and computes descriptors; one elected lane issues (see the producer)
      const bool elected = elect_one();
      const uint32_t idesc_s = instr_desc(TC_BK, 0), idesc_o = instr_desc(D, 1);
      const uint32_t q_addr = smem_u32(q_sm + t * Q_BYTES), p_addr = smem_u32(p_sm + t * P_BYTES);
      // S = Q K^T: k runs over the head in steps of 16 (32 bytes inside a 128-byte chunk)
      auto issue_s = [&](int buf) {
        if (elected) {
#pragma unroll
          for (int k = 0; k < D / 16; ++k) {
            const uint32_t off = (k >> 2) * SUB + (k & 3) * 32;
            umma_bf16(tmem_base + t * TC_BK, smem_desc(q_addr + off, 16),
                      smem_desc(smem_u32(ring + buf * KV_BYTES) + off, 16), idesc_s, k > 0 ? 1u : 0u);
          }
          umma_commit(&s_ready[t]);
        }
      };
      // O (+)= P V: k runs over the 128 keys in steps of 16; P K-major (two 64-key chunks); V's
      // rows are keys (16 keys = 2048 bytes), its 64-wide chunks of the head are SUB bytes apart
      auto issue_pv = [&](bool first) {
        if (elected) {
#pragma unroll
          for (int k = 0; k < TC_BK / 16; ++k) {
            const uint32_t a_off = (k >> 2) * SUB + (k & 3) * 32;
            umma_bf16(tmem_base + 2 * TC_BK + t * 128, smem_desc(p_addr + a_off, 16),
                      smem_desc(smem_u32(ring + 2 * KV_BYTES) + k * 2048, SUB), idesc_o,
                      (first && k == 0) ? 0u : 1u);
          }
          umma_commit(&o_ready[t]);
        }
      };
      // A buffer is free after two arrivals, one per tile; a tile that is alone in a step makes both.
      auto release = [&](int buf, bool alone) {
        if (elected) {
          umma_commit(&empty[buf]);
          if (alone) umma_commit(&empty[buf]);
        }
        __syncwarp();
      };
      // every lane waits; the warp goes on together or stops together
      auto wait2 = [&](uint64_t* first_bar, uint32_t first_parity, uint64_t* second_bar, uint32_t second_parity) -> bool {
        const bool got = mbar_wait(first_bar, first_parity, abort) && mbar_wait(second_bar, second_parity, abort);
        return __all_sync(0xffffffffu, got);
      };
      bool ok = wait2(&q_full, 0, &full[0], 0);
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        issue_s(0);
        release(0, n_other == 0);
      }
      // Step i: S of step i+1 as soon as the softmax warps have read S of step i out of tensor
      // memory (they are still busy with its exponentials), then PV of step i when P is written.
      for (int i = 0; i < n_mine && ok; ++i) {
        if (i + 1 < n_mine) {
          const int kb = (i + 1) & 1;                  // buffer of K(i+1); V(i) is in buffer 2
          ok = wait2(&full[kb], ((i + 1) >> 1) & 1, &s_free[t], i & 1);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_s(kb);
          release(kb, i + 1 >= n_other);
        }
        ok = wait2(&full[2], i & 1, &p_ready[t], i & 1);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        issue_pv(i == 0);
        release(2, i >= n_other);
      }
    }
  } else if (warp < 8) {
    // ---------------- softmax and output: warps 0-3 own tile 0, warps 4-7 tile 1; thread = query
    // row = TMEM lane.  The running output stays in tensor memory; it is rescaled only when a row's
    // maximum has grown by more than 2^8 since the last rescale, so most steps only produce P.
    const int t = warp >> 2;
    const int quarter = warp & 3;
    const int r = quarter * 32 + lane;
    const int pos = pos0 + t * TC_BQ + r;
    const uint32_t lane_addr = (uint32_t)(quarter * 32) << 16;
    const uint32_t tmem_s = tmem_base + t * TC_BK + lane_addr;
    const uint32_t tmem_o = tmem_base + 2 * TC_BK + t * 128 + lane_addr;
    uint8_t* p_row = p_sm + t * P_BYTES + r * 128;
    const int n_mine = n_tile[t];
    float m_ref = -INFINITY, l_run = 0.f;
    pdl_wait();
    bool ok = true;
    for (int i = 0; i < n_mine && ok; ++i) {
      ok = mbar_wait(&s_ready[t], i & 1, abort);
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const int j0 = (page_lo + 2 * i) * SB_PAGE_TOKENS;
      const bool edge = j0 + TC_BK - 1 > pos0 + t * TC_BQ ||
                        (window > 0 && j0 <= pos0 + t * TC_BQ + TC_BQ - window);
      float sv[64];
      uint32_t pk[32];
      float mx = -INFINITY, rs = 0.f, rs_hi = 0.f;   // the row sum in two halves (packed adds)
      float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      // half h of the row of S from tensor memory, masked where the step touches an edge
      auto load_half = [&](int h) {
        tmem_load64(tmem_s + h * 64, sv);
        if (edge) {
#pragma unroll
          for (int e = 0; e < 64; ++e) {
            const int j = j0 + h * 64 + e;
            if (j > pos || (window > 0 && j <= pos - window)) sv[e] = -INFINITY;
          }
        }
      };
      // P = exp2(S * scale - m) of 8 keys, rounded to bfloat16: one 16-byte column of the A operand
      auto exp8 = [&](int c, uint32_t* w) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float x0, x1;
          fma2(x0, x1, sv[c * 8 + 2 * e], sv[c * 8 + 2 * e + 1], scale_log2, -m_use);
          const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
          add2(rs, rs_hi, p0, p1);
          __nv_bfloat162 two = __floats2bfloat162_rn(p0, p1);
          w[e] = *reinterpret_cast<uint32_t*>(&two);
        }
      };
      // K-major A operand: 64-key chunk h, 16-byte column c ^ (r % 8) of row r
      auto store8 = [&](int h, int c, const uint32_t* w) {
        *reinterpret_cast<uint4*>(p_row + h * SUB + ((c ^ (r & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      };
      auto s_consumed = [&]() {                        // S of this step may be overwritten
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(&s_free[t]);
      };
      // One pass in the common case: the exponent's reference is the one of the step before, which
      // is good as long as no row's maximum outgrows it by more than 2^8.
      load_half(0);
#pragma unroll
      for (int e = 0; e < 64; ++e) mx = fmaxf(mx, sv[e]);
#pragma unroll
      for (int c = 0; c < 8; ++c) exp8(c, pk + 4 * c);
      load_half(1);
#pragma unroll
      for (int e = 0; e < 64; ++e) mx = fmaxf(mx, sv[e]);
      mx *= scale_log2;                               // scale_log2 > 0: the maximum commutes with it
      const bool outgrown = mx > m_ref + 8.f;         // also the first keys a row sees (m_ref = -inf)
      if (!__any_sync(0xffffffffu, outgrown)) {
        s_consumed();
        // P's tile and O are free once PV of the step before has finished
        if (i > 0) ok = mbar_wait(&o_ready[t], (i - 1) & 1, abort);
        if (!ok) break;
#pragma unroll
        for (int c = 0; c < 8; ++c) store8(0, c, pk + 4 * c);
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t w[4];
          exp8(c, w);
          store8(1, c, w);
        }
      } else {
        // a new reference: rescale what has been accumulated, then redo this step's P
        const float m_new = fmaxf(m_ref, mx);
        const float alpha = m_ref == -INFINITY ? 1.f : fast_exp2(m_ref - m_new);
        if (i > 0) {
          ok = mbar_wait(&o_ready[t], (i - 1) & 1, abort);
          if (!ok) break;
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
          for (int c = 0; c < D; c += 32) {
            float ov[32];
            tmem_load32(tmem_o + c, ov);
#pragma unroll
            for (int e = 0; e < 32; ++e) ov[e] *= alpha;
            tmem_store32(tmem_o + c, ov);
          }
          asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
        }
        l_run *= alpha;
        m_ref = m_new;
        m_use = m_ref == -INFINITY ? 0.f : m_ref;
        rs = 0.f;
        rs_hi = 0.f;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t w[4];
          exp8(c, w);
          store8(1, c, w);
        }
        load_half(0);
        s_consumed();
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          uint32_t w[4];
          exp8(c, w);
          store8(0, c, w);
        }
      }
      l_run += rs + rs_hi;
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_ready[t]);
    }
    if (ok && n_mine > 0) ok = mbar_wait(&o_ready[t], (n_mine - 1) & 1, abort);
    if (ok && n_mine > 0) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const float inv = 1.f / l_run;
      const bool valid = t * TC_BQ + r < rows_valid;
      bf16* dst = out + ((size_t)seq_q_start[seq] + q_first + t * TC_BQ + r) * ((size_t)heads * D) + (size_t)head * D;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        float ov[32];
        tmem_load32(tmem_o + c, ov);
        if (valid) {
#pragma unroll
          for (int d = 0; d < 32; d += 8) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              __nv_bfloat162 pk = __floats2bfloat162_rn(ov[d + 2 * e] * inv, ov[d + 2 * e + 1] * inv);
              w[e] = *reinterpret_cast<uint32_t*>(&pk);
            }
            *reinterpret_cast<uint4*>(dst + c + d) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
  }

  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 9) {
    __syncwarp();
    tmem_free(tmem_holder, TMEM_COLS);
  }
  if (threadIdx.x == 0 && abort_flag && status) atomicOr(status, 16);
}

// ------------------------------------------------------------------------------------------ host

template <int D>
static int launch(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, void* out,
                  const int* block_table, int table_stride, const int* seq_slot, const int* seq_q_start,
                  const int* seq_q_len, const int* seq_kv_len, const int* tile_seq, const int* tile_first,
                  int n_tiles, int heads, int kv_heads, float scale, int window, int* status, int list_of_blocks,
                  cudaStream_t s) {
  constexpr int DC = D / 64;
  const int smem = (2 * DC + 4 + TC_RING * DC) * 128 * 128 + 1024;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_prefill_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    configured = true;
  }
  return launch_dependent(attention_prefill_tc_kernel<D>, dim3(heads, n_tiles), dim3(TC_THREADS), smem, s, mq, mk,
                          mv, (bf16*)out, block_table, table_stride, seq_slot, seq_q_start, seq_q_len, seq_kv_len,
                          tile_seq, tile_first, heads, kv_heads, scale * 1.4426950408889634f, window, status,
                          list_of_blocks);
}

static unsigned long long next_limit_ns = WAIT_LIMIT_NS;
static int next_withhold_step = -1;

extern "C" {

// For tests of the give-up path: the NEXT sb_attention_prefill_tc launch leaves out half of the
// values of step `step` (128 keys) of every block and its waits give up after `limit_ns`.  The
// blocks cannot finish; the launch must return with bit 16 of *status set.  The switches are set
// and put back by copies on the launch's stream, around that one launch.
void sb_attention_prefill_tc_withhold(int step, unsigned long long limit_ns) {
  next_withhold_step = step;
  next_limit_ns = limit_ns ? limit_ns : WAIT_LIMIT_NS;
}

// Same contract as sb_attention_prefill; n_tokens rows in q/out, n_pages pages in the stores.
// list_of_blocks: tile_seq/tile_first list blocks of 256 queries (else tiles of 64, see the kernel).
// head_dim must be 64 or 128 (returns -2 otherwise).
int sb_attention_prefill_tc(const void* q, void* out, const void* k_store, const void* v_store,
                            const int* block_table, int table_stride, const int* seq_slot,
                            const int* seq_q_start, const int* seq_q_len, const int* seq_kv_len,
                            const int* tile_seq, const int* tile_first, int n_tiles, int n_tokens,
                            int n_pages, int heads, int kv_heads, int head_dim, float scale, int window,
                            int* status, int list_of_blocks, cudaStream_t s) {
  if (n_tiles == 0) return 0;
  if (kv_heads <= 0 || heads % kv_heads) return -2;
  if (head_dim != 64 && head_dim != 128) return -2;
  if (((uintptr_t)q | (uintptr_t)out | (uintptr_t)k_store | (uintptr_t)v_store) & 15) return -2;
  CUtensorMap mq, mk, mv;
  int rc = sb_make_map(&mq, q, n_tokens, (long long)heads * head_dim, TC_BQ);
  if (rc) return rc;
  const long long kv_rows = (long long)n_pages * kv_heads * SB_PAGE_TOKENS;
  rc = sb_make_map(&mk, k_store, kv_rows, head_dim, SB_PAGE_TOKENS);
  if (rc) return rc;
  rc = sb_make_map(&mv, v_store, kv_rows, head_dim, SB_PAGE_TOKENS);
  if (rc) return rc;
#define ARGS mq, mk, mv, out, block_table, table_stride, seq_slot, seq_q_start, seq_q_len, seq_kv_len, \
             tile_seq, tile_first, n_tiles, heads, kv_heads, scale, window, status, list_of_blocks, s
  const bool test_run = next_withhold_step >= 0;
  if (test_run) {
    cudaMemcpyToSymbolAsync(tc_withhold_step, &next_withhold_step, sizeof(int), 0, cudaMemcpyHostToDevice, s);
    cudaMemcpyToSymbolAsync(tc_wait_limit_ns, &next_limit_ns, sizeof(next_limit_ns), 0, cudaMemcpyHostToDevice, s);
    cudaStreamSynchronize(s);
  }
  rc = head_dim == 64 ? launch<64>(ARGS) : launch<128>(ARGS);
  if (test_run) {
    cudaStreamSynchronize(s);
    next_withhold_step = -1;
    next_limit_ns = WAIT_LIMIT_NS;
    cudaMemcpyToSymbolAsync(tc_withhold_step, &next_withhold_step, sizeof(int), 0, cudaMemcpyHostToDevice, s);
    cudaMemcpyToSymbolAsync(tc_wait_limit_ns, &next_limit_ns, sizeof(next_limit_ns), 0, cudaMemcpyHostToDevice, s);
    cudaStreamSynchronize(s);
  }
  return rc;
#undef ARGS
}

}  // extern "C"
