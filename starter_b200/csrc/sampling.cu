// Token selection from float logits: greedy argmax, or a draw from softmax(logits / temperature).
//
// Greedy keeps the lowest index among equal maxima (engine/engine.py:833 uses argmax).  The draw uses
// the Gumbel-max identity: argmax_i(logit_i / t + g_i) with g_i = -log(-log(u_i)) is distributed as
// softmax(logits / t), so sampling is one more argmax and needs no normalisation pass.  u_i comes from
// a counter-based hash of (row key, vocabulary index); the row key is derived from the sampling seed,
// the request's own number and the position of the token being drawn, so a request draws the same
// tokens whatever else is in its batch.  The host-side statement of the same arithmetic is
// starter_b200/sampling/sampler.py:gumbel_noise.
#include "common.cuh"

__host__ __device__ __forceinline__ uint32_t sb_mix32(uint32_t x) {
  x ^= x >> 16;
  x *= 0x7feb352du;
  x ^= x >> 15;
  x *= 0x846ca68bu;
  x ^= x >> 16;
  return x;
}

#define SAMPLE_CHUNK 4096

struct Best { float v; int i; };

__device__ __forceinline__ Best better(Best a, Best b) {
  return (b.v > a.v || (b.v == a.v && b.i < a.i)) ? b : a;
}

__device__ __forceinline__ Best block_best(Best b, float* sh_v, int* sh_i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    Best other = {__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
    b = better(b, other);
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { sh_v[warp] = b.v; sh_i[warp] = b.i; }
  __syncthreads();
  if (warp == 0) {
    const int warps = blockDim.x >> 5;
    b.v = lane < warps ? sh_v[lane] : -INFINITY;
    b.i = lane < warps ? sh_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      Best other = {__shfl_xor_sync(0xffffffffu, b.v, o), __shfl_xor_sync(0xffffffffu, b.i, o)};
      b = better(b, other);
    }
  }
  return b;  // valid in warp 0
}

// Stage 1: block (chunk, row) finds the best candidate among SAMPLE_CHUNK logits of its row.
__global__ void sample_chunk_kernel(const float* __restrict__ logits, int vocab, size_t row_stride,
                                    const float* __restrict__ temperature,
                                    const uint32_t* __restrict__ request_key, const int* position,
                                    float* __restrict__ cand_v, int* __restrict__ cand_i) {
  __shared__ float sh_v[32];
  __shared__ int sh_i[32];
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(logits);
  SB_BEHIND_WAIT(temperature);
  SB_BEHIND_WAIT(request_key);
  const int row = blockIdx.y, chunk = blockIdx.x;
  const float* lr = logits + (size_t)row * row_stride;
  const float t = temperature ? temperature[row] : 0.f;
  const bool greedy = !(t > 0.f);
  const float inv_t = greedy ? 1.f : 1.f / t;
  uint32_t row_key = 0;
  if (!greedy) row_key = sb_mix32((uint32_t)position[row] + sb_mix32(request_key[row]));
  Best b = {-INFINITY, 0x7fffffff};
  const int end = min(vocab, (chunk + 1) * SAMPLE_CHUNK);
  for (int i = chunk * SAMPLE_CHUNK + threadIdx.x; i < end; i += blockDim.x) {
    float v = lr[i] * inv_t;
    if (!greedy) {
      const uint32_t r = sb_mix32((uint32_t)i ^ row_key);
      const float u = ((float)(r >> 8) + 0.5f) * (1.0f / 16777216.0f);
      v += -logf(-logf(u));
    }
    Best c = {v, i};
    b = better(b, c);
  }
  b = block_best(b, sh_v, sh_i);
  if (threadIdx.x == 0) {
    cand_v[(size_t)row * gridDim.x + chunk] = b.v;
    cand_i[(size_t)row * gridDim.x + chunk] = b.i;
  }
}

// Stage 2: one block per row picks among the chunk candidates.
__global__ void sample_pick_kernel(const float* __restrict__ cand_v, const int* __restrict__ cand_i,
                                   int chunks, int vocab, int* __restrict__ out, int* status,
                                   int* feed_token, int* feed_pos, int* feed_len) {
  __shared__ float sh_v[32];
  __shared__ int sh_i[32];
  pdl_trigger();
  pdl_wait();
  SB_BEHIND_WAIT(cand_v);
  SB_BEHIND_WAIT(cand_i);
  const int row = blockIdx.x;
  Best b = {-INFINITY, 0x7fffffff};
  for (int c = threadIdx.x; c < chunks; c += blockDim.x) {
    Best o = {cand_v[(size_t)row * chunks + c], cand_i[(size_t)row * chunks + c]};
    b = better(b, o);
  }
  b = block_best(b, sh_v, sh_i);
  if (threadIdx.x == 0) {
    int bi = b.i;
    if (bi < 0 || bi >= vocab) {  // every logit was NaN
      if (status) atomicOr(status, 2);
      bi = 0;
    }
    out[row] = bi;
    // self-feeding decode: the drawn token becomes the row's next input, one position further on
    // (engine/engine.py:835-838).  Stage 1, which reads position[row], has finished.
    if (feed_token) {
      feed_token[row] = bi;
      feed_pos[row] += 1;
      feed_len[row] += 1;
    }
  }
}

extern "C" {

int sb_sample_chunks(int vocab) { return (vocab + SAMPLE_CHUNK - 1) / SAMPLE_CHUNK; }

// logits: [rows, vocab] float with `row_stride` floats between rows.  temperature may be null (all
// greedy); rows with temperature <= 0 are greedy.  request_key and position are read only for rows
// that draw.  cand_v / cand_i: scratch of rows * sb_sample_chunks(vocab) entries each.  With
// feed_token (all three feed arrays or none), row r also stores its token in feed_token[r] and adds
// one to feed_pos[r] and feed_len[r]; position may alias feed_len.
int sb_sample(const float* logits, int rows, int vocab, long long row_stride, const float* temperature,
              const uint32_t* request_key, const int* position, int* out, int* status,
              int* feed_token, int* feed_pos, int* feed_len, float* cand_v, int* cand_i,
              cudaStream_t s) {
  if (rows == 0) return 0;
  const int chunks = sb_sample_chunks(vocab);
  int rc = launch_dependent(sample_chunk_kernel, dim3(chunks, rows), dim3(256), 0, s, logits, vocab,
                            (size_t)row_stride, temperature, request_key, position, cand_v, cand_i);
  if (rc) return rc;
  return launch_dependent(sample_pick_kernel, dim3(rows), dim3(128), 0, s, (const float*)cand_v,
                          (const int*)cand_i, chunks, vocab, out, status, feed_token, feed_pos, feed_len);
}

}  // extern "C"
