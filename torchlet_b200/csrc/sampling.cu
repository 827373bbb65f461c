// Token selection over float32 logits [rows, vocab], one block per row.
//
// temperature == 0: argmax, the lowest index wins a tie (the reference samples with
// logits.argmax only, v10_triton_paged_gqa/engine.py:187-188).
// temperature  > 0: a draw from softmax(logits / temperature) by the Gumbel-max rule:
// argmax_i (logits_i / temperature - log(-log(u_i))), with u_i in (0, 1) from a
// counter-based generator keyed by (seed, counter, i).  The draw of a request
// therefore depends only on its own seed and on how many tokens it has sampled, not
// on the batch it is in.
#include <math.h>

#include "common.cuh"
#include "sampling_static.h"

namespace {

__device__ __forceinline__ unsigned long long mix64(unsigned long long x) {
  x ^= x >> 30;
  x *= 0xBF58476D1CE4E5B9ull;
  x ^= x >> 27;
  x *= 0x94D049BB133111EBull;
  x ^= x >> 31;
  return x;
}

__device__ __forceinline__ float uniform_for(unsigned long long key, int index) {
  const unsigned long long bits = mix64(key ^ ((unsigned long long)(index + 1) * 0xD1B54A32D192ED03ull));
  return ((float)(bits >> 41) + 0.5f) * (1.0f / 8388608.0f);  // exact in float32, never 0 or 1
}

constexpr int NT = 1024;
constexpr int CHUNK = 8192;  // vocabulary entries one block scans when a row is split

struct Best {
  float value;
  int index;
};

__device__ __forceinline__ bool better(float v, int i, float bv, int bi) {
  return v > bv || (v == bv && i < bi);
}

// Best (value, lowest index) over a block; valid in thread 0.
__device__ __forceinline__ Best block_best(float bv, int bi) {
  __shared__ float best_v[NT / 32];
  __shared__ int best_i[NT / 32];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) {
      bv = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) {
    best_v[warp] = bv;
    best_i[warp] = bi;
  }
  __syncthreads();
  if (warp == 0) {
    const int warps = blockDim.x >> 5;
    bv = lane < warps ? best_v[lane] : -INFINITY;
    bi = lane < warps ? best_i[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (better(ov, oi, bv, bi)) {
        bv = ov;
        bi = oi;
      }
    }
  }
  return Best{bv, bi};
}

// Block (row r, chunk c) scans vocabulary entries [c * span, (c + 1) * span) of row r.
// gridDim.y == 1: writes the token; else writes its best to scratch[r][c].
__global__ void __launch_bounds__(NT)
sample_kernel(const float* __restrict__ logits, size_t row_stride, int vocab, int span,
              const float* __restrict__ temperature, const long long* __restrict__ seed,
              const int* __restrict__ counter, int* __restrict__ out, Best* __restrict__ scratch) {
  tl::pdl_wait();               // everything before us in the stream is complete and visible
  tl::pdl_launch_dependents();  // the next kernel may start its own prologue

  const int r = blockIdx.x;
  const float* row = logits + (size_t)r * row_stride;
  const float temp = temperature ? temperature[r] : 0.f;
  unsigned long long key = 0;
  if (temp > 0.f)
    key = mix64((unsigned long long)seed[r] * 0x9E3779B97F4A7C15ull + (unsigned long long)counter[r] +
                0x632BE59BD9B4E019ull);
  const float inv_temp = temp > 0.f ? 1.f / temp : 1.f;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  const int begin = blockIdx.y * span, end = min(vocab, begin + span);
  for (int i = begin + threadIdx.x; i < end; i += NT) {
    float v = row[i];
    if (temp > 0.f) v = v * inv_temp - logf(-logf(uniform_for(key, i)));
    if (better(v, i, bv, bi) || bi == 0x7fffffff) {
      bv = v;
      bi = i;
    }
  }
  const Best best = block_best(bv, bi);
  if (threadIdx.x == 0) {
    if (gridDim.y == 1)
      out[r] = best.index == 0x7fffffff ? 0 : best.index;
    else
      scratch[(size_t)r * gridDim.y + blockIdx.y] = best;
  }
}

__global__ void sample_merge_kernel(const Best* __restrict__ scratch, int chunks, int* __restrict__ out) {
  tl::pdl_wait();               // everything before us in the stream is complete and visible
  tl::pdl_launch_dependents();  // the next kernel may start its own prologue

  const int r = blockIdx.x, lane = threadIdx.x;
  float bv = -INFINITY;
  int bi = 0x7fffffff;
  for (int c = lane; c < chunks; c += 32) {
    const Best b = scratch[(size_t)r * chunks + c];
    if (better(b.value, b.index, bv, bi)) {
      bv = b.value;
      bi = b.index;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (better(ov, oi, bv, bi)) {
      bv = ov;
      bi = oi;
    }
  }
  if (lane == 0) out[r] = bi == 0x7fffffff ? 0 : bi;
}

}  // namespace

extern "C" {

// Bytes of scratch that let a row be scanned by several blocks (0: one block a row).
long long tl_sample_scratch_bytes(int rows, int vocab) {
  const long long chunks = ((long long)vocab + CHUNK - 1) / CHUNK;
  return chunks > 1 ? (long long)rows * chunks * (long long)sizeof(Best) : 0;
}

int tl_sample(const float* logits, long long row_stride, int rows, int vocab, const float* temperature,
              const long long* seed, const int* counter, int* out, void* scratch, long long scratch_bytes,
              cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || !logits || !out) return TL_ERR_UNSUPPORTED;
  // a row with temperature > 0 reads its seed and its counter: all three, or none
  if (temperature && (!seed || !counter)) return TL_ERR_UNSUPPORTED;
  long long chunks = ((long long)vocab + CHUNK - 1) / CHUNK;
  if (chunks > 1 && (!scratch || scratch_bytes < tl_sample_scratch_bytes(rows, vocab))) chunks = 1;
  if (chunks > 65535) return TL_ERR_UNSUPPORTED;
  const int span = chunks > 1 ? CHUNK : vocab;
  tl::launch_kernel(sample_kernel, dim3(rows, (unsigned)chunks), NT, 0, stream, logits, (size_t)row_stride, vocab, span,
                    temperature, seed, counter, out, (Best*)scratch);
  int rc = TL_LAUNCH_CHECK();
  if (rc || chunks == 1) return rc;
  tl::launch_kernel(sample_merge_kernel, rows, 32, 0, stream, (const Best*)scratch, (int)chunks, out);
  return TL_LAUNCH_CHECK();
}

// ---------------------------------------------------------------------------
// The variant that allocates nothing (see sampling_static.h).  The partial results of
// the blocks that share a row live in this array instead of a caller's buffer.
static __device__ __align__(256) Best g_static_partials[TL_SAMPLE_STATIC_MAX_PARTIALS];

int tl_sample_static(const float* logits, long long row_stride, int rows, int vocab, const float* temperature,
                     const long long* seed, const int* counter, int* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0 || !logits || !out) return TL_ERR_UNSUPPORTED;
  // a row with temperature > 0 reads its seed and its counter: all three, or none
  if (temperature && (!seed || !counter)) return TL_ERR_UNSUPPORTED;
  const long long chunks = ((long long)vocab + CHUNK - 1) / CHUNK;
  if (chunks > 65535 || (long long)rows * chunks > TL_SAMPLE_STATIC_MAX_PARTIALS) return TL_SAMPLE_STATIC_TOO_LARGE;
  // In host code the array's name is only a stand-in: the device address is looked up
  // once per device, with that device current, and kept.
  constexpr int MAX_DEVICES = 64;
  static Best* partials_on[MAX_DEVICES] = {};
  int device = 0;
  cudaError_t err = cudaGetDevice(&device);
  if (err != cudaSuccess) return (int)err;
  if (device < 0 || device >= MAX_DEVICES) return TL_ERR_UNSUPPORTED;
  if (!partials_on[device]) {
    void* address = nullptr;
    err = cudaGetSymbolAddress(&address, g_static_partials);
    if (err != cudaSuccess) return (int)err;
    partials_on[device] = static_cast<Best*>(address);
  }
  Best* partials = partials_on[device];
  const int span = chunks > 1 ? CHUNK : vocab;
  tl::launch_kernel(sample_kernel, dim3(rows, (unsigned)chunks), NT, 0, stream, logits, (size_t)row_stride, vocab,
                    span, temperature, seed, counter, out, partials);
  int rc = TL_LAUNCH_CHECK();
  if (rc || chunks == 1) return rc;
  tl::launch_kernel(sample_merge_kernel, rows, 32, 0, stream, (const Best*)partials, (int)chunks, out);
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
