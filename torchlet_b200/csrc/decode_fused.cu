// Finishing kernels of the decode path.  With few tokens the tensor-core product runs
// "swapped" with its K dimension split over CTAs and leaves float32 partial sums
// [splits][tokens][N] (see gemm_tc.cu).  Instead of a generic finishing pass followed by
// another small kernel, the partials are consumed by the operation that comes next:
//
//   finish_qkv_rope   : sum of the splits + bias -> rotary encoding of q and k by position
//                       -> q to the activation buffer, k and v to their cache pages
//                       (replaces: split finish, rope_kv_kernel);
//   finish_accum_norm : sum of the splits (+ bias) added into the float32 residual stream,
//                       then RMSNorm of the updated row into the compute dtype
//                       (replaces: split finish, rms_norm_kernel).
//
// Sums run over the splits in ascending order, in float32; angles, rotation, the residual
// sum and the norm are float32 (the same formulas as elementwise.cu).
#include "common.cuh"

namespace {

using namespace tl;

__global__ void finish_qkv_rope_kernel(const float* __restrict__ partial, int splits,
                                       const float* __restrict__ bias, __nv_bfloat16* __restrict__ qkv,
                                       const int* __restrict__ positions, const int* __restrict__ token_req,
                                       const int* __restrict__ block_table, int table_width,
                                       __nv_bfloat16* __restrict__ pages, const float* __restrict__ inv_freq,
                                       int tokens, int nh, int nkv, int d, int page_size, int write_kv,
                                       int num_pages) {
  tl::pdl_launch_dependents();  // the next kernel may start its prologue (it waits for us before it reads our output)
  tl::pdl_wait();               // everything before us in the stream is complete and visible

  const int t = blockIdx.x, h = blockIdx.y;
  const int half = d >> 1;
  const int N = (nh + 2 * nkv) * d;
  const size_t plane = (size_t)tokens * N;
  const int pos = positions[t];
  const bool is_v = h >= nh + nkv;
  __nv_bfloat16* dst = qkv + (size_t)t * N + (size_t)h * d;
  if (h >= nh) {
    if (!write_kv) return;
    const int kvh = is_v ? h - nh - nkv : h - nh;
    if (!TL_DEBUG_OK(pos >= 0 && pos / page_size < table_width, TL_DEBUG_POSITION, pos)) return;
    const int page = block_table[(size_t)token_req[t] * table_width + pos / page_size];
    if (!TL_DEBUG_OK(page >= 0 && page < num_pages, TL_DEBUG_PAGE, page)) return;
    dst = pages + ((((size_t)page * 2 + (is_v ? 1 : 0)) * nkv + kvh) * page_size + pos % page_size) * d;
  }
  const float* src = partial + (size_t)t * N + (size_t)h * d;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float x1 = bias ? bias[h * d + i] : 0.f, x2 = bias ? bias[h * d + i + half] : 0.f;
    // all splits of the pair are requested before the first is added (up to 16 at a time): the
    // kernel's time is its trips to L2
    for (int s0 = 0; s0 < splits; s0 += 16) {
      float a[16], b[16];
#pragma unroll
      for (int s = 0; s < 16; ++s) {
        const bool live = s0 + s < splits;
        a[s] = live ? src[(size_t)(s0 + s) * plane + i] : 0.f;
        b[s] = live ? src[(size_t)(s0 + s) * plane + i + half] : 0.f;
      }
#pragma unroll
      for (int s = 0; s < 16; ++s) {  // ascending splits; past the last one zeros are added
        x1 += a[s];
        x2 += b[s];
      }
    }
    // the product's output is bfloat16 in the unfused path: round here too, so that both
    // paths give the same numbers
    x1 = __bfloat162float(__float2bfloat16_rn(x1));
    x2 = __bfloat162float(__float2bfloat16_rn(x2));
    if (is_v) {
      dst[i] = __float2bfloat16_rn(x1);
      dst[i + half] = __float2bfloat16_rn(x2);
    } else {
      float sn, cs;
      sincosf((float)pos * inv_freq[i], &sn, &cs);
      dst[i] = __float2bfloat16_rn(x1 * cs - x2 * sn);
      dst[i + half] = __float2bfloat16_rn(x2 * cs + x1 * sn);
    }
  }
}

// One block per token row.  PER = elements of the row each thread keeps in registers.
template <int NT, int PER>
__global__ void __launch_bounds__(NT)
finish_accum_norm_kernel(const float* __restrict__ partial, int splits, const float* __restrict__ bias,
                         float* __restrict__ acc, const float* __restrict__ weight,
                         __nv_bfloat16* __restrict__ out, int tokens, int hidden, float eps) {
  tl::pdl_launch_dependents();  // the next kernel may start its prologue (it waits for us before it reads our output)
  tl::pdl_wait();               // everything before us in the stream is complete and visible

  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const size_t plane = (size_t)tokens * hidden;
  float* row = acc + (size_t)t * hidden;
  const float* src = partial + (size_t)t * hidden;
  // loads are issued PER at a time (one per register), so their latencies overlap
  float v[PER], sum[PER];
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int j = threadIdx.x + k * NT;
    v[k] = j < hidden ? row[j] : 0.f;
    sum[k] = (bias && j < hidden) ? bias[j] : 0.f;
  }
  int s = 0;
  for (; s + 2 <= splits; s += 2) {  // two splits a round: 2 * PER loads in flight
    float part0[PER], part1[PER];
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int j = threadIdx.x + k * NT;
      part0[k] = j < hidden ? src[s * plane + j] : 0.f;
      part1[k] = j < hidden ? src[(s + 1) * plane + j] : 0.f;
    }
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      sum[k] += part0[k];
      sum[k] += part1[k];
    }
  }
  for (; s < splits; ++s) {
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int j = threadIdx.x + k * NT;
      sum[k] += j < hidden ? src[s * plane + j] : 0.f;
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int j = threadIdx.x + k * NT;
    v[k] += sum[k];
    if (j < hidden) row[j] = v[k];
    ss = fmaf(v[k], v[k], ss);
  }
  ss = block_sum<NT>(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  if (out) {
#pragma unroll
    for (int k = 0; k < PER; ++k) {
      const int j = threadIdx.x + k * NT;
      if (j < hidden) out[(size_t)t * hidden + j] = __float2bfloat16_rn(v[k] * inv * weight[j]);
    }
  }
}

}  // namespace

TL_DEBUG_READER(tl_decode_fused_debug_error)

extern "C" {

int tl_finish_qkv_rope(const float* partial, int splits, const float* bias, void* qkv, const int* positions,
                       const int* token_req, const int* block_table, int table_width, void* pages,
                       const float* inv_freq, int tokens, int nh, int nkv, int d, int page_size, int write_kv,
                       int num_pages, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (d % 2 || splits < 1) return TL_ERR_UNSUPPORTED;
  const int heads = write_kv ? nh + 2 * nkv : nh;
  if (heads > 65535) return TL_ERR_UNSUPPORTED;
  int nt = ((d / 2 + 31) / 32) * 32;
  if (nt > 128) nt = 128;
  tl::launch_kernel(finish_qkv_rope_kernel, dim3(tokens, heads), nt, 0, stream, 
      partial, splits, bias, (__nv_bfloat16*)qkv, positions, token_req, block_table, table_width,
      (__nv_bfloat16*)pages, inv_freq, tokens, nh, nkv, d, page_size, write_kv, num_pages);
  return TL_LAUNCH_CHECK();
}

// acc[t] += sum of splits (+ bias); out[t] = rmsnorm(acc[t]) * weight (out may be null:
// only the residual stream is updated).  hidden up to 16384.
int tl_finish_accum_norm(const float* partial, int splits, const float* bias, float* acc, const float* weight,
                         void* out, int tokens, int hidden, float eps, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (splits < 1 || hidden <= 0) return TL_ERR_UNSUPPORTED;
  __nv_bfloat16* o = (__nv_bfloat16*)out;
  if (hidden <= 1024)
    tl::launch_kernel(finish_accum_norm_kernel<256, 4>, tokens, 256, 0, stream, partial, splits, bias, acc, weight, o, tokens, hidden, eps);
  else if (hidden <= 4096)
    tl::launch_kernel(finish_accum_norm_kernel<512, 8>, tokens, 512, 0, stream, partial, splits, bias, acc, weight, o, tokens, hidden, eps);
  else if (hidden <= 16384)
    tl::launch_kernel(finish_accum_norm_kernel<1024, 16>, tokens, 1024, 0, stream, partial, splits, bias, acc, weight, o, tokens, hidden, eps);
  else
    return TL_ERR_UNSUPPORTED;
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
