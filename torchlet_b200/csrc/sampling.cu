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

__global__ void __launch_bounds__(NT)
sample_kernel(const float* __restrict__ logits, size_t row_stride, int vocab,
              const float* __restrict__ temperature, const long long* __restrict__ seed,
              const int* __restrict__ counter, int* __restrict__ out) {
  __shared__ float best_v[NT / 32];
  __shared__ int best_i[NT / 32];
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
  for (int i = threadIdx.x; i < vocab; i += NT) {
    float v = row[i];
    if (temp > 0.f) v = v * inv_temp - logf(-logf(uniform_for(key, i)));
    if (v > bv || (v == bv && i < bi) || bi == 0x7fffffff) {
      bv = v;
      bi = i;
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > bv || (ov == bv && oi < bi)) {
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
    bv = best_v[lane];
    bi = best_i[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) {
        bv = ov;
        bi = oi;
      }
    }
    if (lane == 0) out[r] = bi == 0x7fffffff ? 0 : bi;
  }
}

}  // namespace

extern "C" int tl_sample(const float* logits, long long row_stride, int rows, int vocab,
                         const float* temperature, const long long* seed, const int* counter,
                         int* out, cudaStream_t stream) {
  if (rows <= 0) return 0;
  if (vocab <= 0) return TL_ERR_UNSUPPORTED;
  sample_kernel<<<rows, NT, 0, stream>>>(logits, (size_t)row_stride, vocab, temperature, seed, counter, out);
  return TL_LAUNCH_CHECK();
}
