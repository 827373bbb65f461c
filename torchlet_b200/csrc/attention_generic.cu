// Paged causal grouped-query attention for any batch of (request, next tokens):
// prompt portions with cached context before them and single decoded tokens alike.
// One warp per (token, query head); keys are visited in tiles of 32 consecutive
// ABSOLUTE positions (tile edges at multiples of 32), so the order of every sum
// depends only on the token's position and window, never on how the sequence was cut
// into steps, on the batch, or on the pages used.  Scores, softmax and the weighted
// sum are float32; T is the storage type of queries, pages and output.
//
// This is the true 32-bit kernel and the any-size bfloat16 kernel (head_dim any
// multiple of 8 up to 256, any head counts, any page size).
//
// Reference counterparts: forward_ragged_attention_kernel and
// forward_slot_attention_decode_kernel, v10_triton_paged_gqa/kernel/gqa.py:5-228
// (query head h reads KV head h // g, scale head_dim^-0.5, key allowed iff
// key_pos <= query_pos, online softmax, acc / l).
#include <math.h>

#include "common.cuh"

namespace {

using namespace tl;

constexpr int WARPS = 4;
constexpr int MAX_D = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attention_generic_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ pages,
                         const int* __restrict__ block_table, int table_width,
                         const int* __restrict__ token_req, const int* __restrict__ positions,
                         T* __restrict__ out, int out_stride, int tokens, int nh, int nkv, int d,
                         int page_size, int window, float scale, int num_pages) {
  tl::pdl_wait();               // everything before us in the stream is complete and visible
  tl::pdl_launch_dependents();  // the next kernel may start its own prologue

  __shared__ float qs[WARPS][MAX_D];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long item = (long long)blockIdx.x * WARPS + warp;
  if (item >= (long long)tokens * nh) return;
  const int t = (int)(item / nh), h = (int)(item % nh);
  const int kvh = h / (nh / nkv);
  const int pos = positions[t];
  const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
  const int* table = block_table + (size_t)token_req[t] * table_width;

  const T* qrow = q + (size_t)t * q_stride + (size_t)h * d;
  for (int i = lane; i < d; i += 32) qs[warp][i] = to_float(qrow[i]);
  __syncwarp();

  const size_t page_elems = (size_t)2 * nkv * page_size * d;
  const size_t k_off = (size_t)kvh * page_size * d;
  const size_t v_off = ((size_t)nkv + kvh) * page_size * d;

  float m = -INFINITY, l = 0.f;
  float acc[MAX_D / 32];
#pragma unroll
  for (int c = 0; c < MAX_D / 32; ++c) acc[c] = 0.f;

  for (int start = lo & ~31; start <= pos; start += 32) {
    const int key = start + lane;
    const bool valid = key >= lo && key <= pos;
    float s = -INFINITY;
    size_t row_off = 0;
    if (valid) {
      int page = 0;  // a key whose table entry fails a debug-build check is read from the reserved page 0
      if (TL_DEBUG_OK(key / page_size < table_width, TL_DEBUG_POSITION, key)) page = table[key / page_size];
      if (!TL_DEBUG_OK(page >= 0 && page < num_pages, TL_DEBUG_PAGE, page)) page = 0;
      row_off = (size_t)page * page_elems + (size_t)(key % page_size) * d;
      const T* krow = pages + row_off + k_off;
      float dot = 0.f;
      for (int i = 0; i < d; i += 8) {
        float kv[8];
        load8(krow + i, kv);
#pragma unroll
        for (int j = 0; j < 8; ++j) dot = fmaf(qs[warp][i + j], kv[j], dot);
      }
      s = dot * scale;
    }
    const float new_m = fmaxf(m, warp_max(s));
    const float corr = expf(m - new_m);  // first tile: exp(-inf) = 0
    const float p = valid ? expf(s - new_m) : 0.f;
    l = l * corr + warp_sum(p);
    m = new_m;
#pragma unroll
    for (int c = 0; c < MAX_D / 32; ++c) acc[c] *= corr;
    const int first = lo > start ? lo - start : 0;
    const int last = pos - start < 31 ? pos - start : 31;
    for (int j = first; j <= last; ++j) {
      const float pj = __shfl_sync(0xffffffffu, p, j);
      const size_t off = __shfl_sync(0xffffffffu, (unsigned long long)row_off, j);
      const T* vrow = pages + off + v_off;
#pragma unroll
      for (int c = 0; c < MAX_D / 32; ++c) {
        const int i = lane + 32 * c;
        if (i < d) acc[c] = fmaf(pj, to_float(vrow[i]), acc[c]);
      }
    }
  }
  T* orow = out + (size_t)t * out_stride + (size_t)h * d;
  const float inv = 1.f / l;
#pragma unroll
  for (int c = 0; c < MAX_D / 32; ++c) {
    const int i = lane + 32 * c;
    if (i < d) orow[i] = from_float<T>(acc[c] * inv);
  }
}

}  // namespace

TL_DEBUG_READER(tl_attention_generic_debug_error)

extern "C" int tl_attention_generic(const void* q, int q_stride, const void* pages, int dtype,
                                    const int* block_table, int table_width, const int* token_req,
                                    const int* positions, void* out, int out_stride, int tokens,
                                    int nh, int nkv, int d, int page_size, int window, float scale,
                                    int num_pages, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (d <= 0 || d > MAX_D || d % 8 || nkv <= 0 || nh % nkv || page_size <= 0 || q_stride % 8)
    return TL_ERR_UNSUPPORTED;
  const long long items = (long long)tokens * nh;
  const unsigned blocks = (unsigned)((items + WARPS - 1) / WARPS);
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(attention_generic_kernel<float>, blocks, WARPS * 32, 0, stream, 
        (const float*)q, q_stride, (const float*)pages, block_table, table_width, token_req,
        positions, (float*)out, out_stride, tokens, nh, nkv, d, page_size, window, scale, num_pages);
  else
    tl::launch_kernel(attention_generic_kernel<__nv_bfloat16>, blocks, WARPS * 32, 0, stream, 
        (const __nv_bfloat16*)q, q_stride, (const __nv_bfloat16*)pages, block_table, table_width,
        token_req, positions, (__nv_bfloat16*)out, out_stride, tokens, nh, nkv, d, page_size, window,
        scale, num_pages);
  return TL_LAUNCH_CHECK();
}
