// Row-wise and element-wise kernels: embedding gather, RMSNorm, rotary position
// encoding fused with the write of keys and values into cache pages, SwiGLU.
// All arithmetic is float32; T is the storage type of activations and weights.
//
// Reference counterparts (Triton): v10_triton_paged_gqa/kernel/rms_norm.py:6-22,
// kernel/rope.py:5-41, kernel/kvcache.py:5-50; nn.Embedding in model/qwen2_5.py:56;
// F.silu(g) * u in v08_paged_gqa_py/layer/ffn_swiglu.py:15.
#include "common.cuh"

namespace {

using namespace tl;

// ---------------------------------------------------------------- embedding
// acc[t, :] = float(table[ids[t], :]);  the residual stream starts in float32.
template <typename T>
__global__ void embed_kernel(const T* __restrict__ table, const int* __restrict__ ids,
                             float* __restrict__ acc, int hidden, int vocab) {
  tl::pdl_launch_dependents();  // the next kernel may start its prologue (it waits for us before it reads our output)
  tl::pdl_wait();               // everything before us in the stream is complete and visible

  const int t = blockIdx.x;
  int id = ids[t];
  const bool ok = id >= 0 && id < vocab;
  TL_DEBUG_OK(ok, TL_DEBUG_TOKEN, id);  // (an id outside the vocabulary reads as a zero row either way)
  const T* row = table + (size_t)(ok ? id : 0) * hidden;
  float* out = acc + (size_t)t * hidden;
  for (int j = threadIdx.x; j < hidden; j += blockDim.x) out[j] = ok ? to_float(row[j]) : 0.f;
}

// ------------------------------------------------------------------ RMSNorm
// out[r, :] = acc[row(r), :] * rsqrt(mean(acc[row(r), :]^2) + eps) * w
// row(r) = rows ? rows[r] : r.  One block per row; the order of the additions
// depends only on the width, never on which other rows are in the batch.
template <typename T, int NT>
__global__ void __launch_bounds__(NT)
rms_norm_kernel(const float* __restrict__ acc, const float* __restrict__ w, const int* __restrict__ rows,
                T* __restrict__ out, int hidden, float eps) {
  tl::pdl_launch_dependents();  // the next kernel may start its prologue (it waits for us before it reads our output)
  tl::pdl_wait();               // everything before us in the stream is complete and visible

  __shared__ float scratch[32];
  constexpr int PER = 8;  // elements a thread keeps in registers; longer rows are re-read
  const int r = blockIdx.x;
  const float* x = acc + (size_t)(rows ? rows[r] : r) * hidden;
  float v[PER];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int j = threadIdx.x + k * NT;
    v[k] = j < hidden ? x[j] : 0.f;
    ss = fmaf(v[k], v[k], ss);
  }
  for (int j = threadIdx.x + PER * NT; j < hidden; j += NT) {
    const float e = x[j];
    ss = fmaf(e, e, ss);
  }
  ss = block_sum<NT>(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  T* o = out + (size_t)r * hidden;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int j = threadIdx.x + k * NT;
    if (j < hidden) o[j] = from_float<T>(v[k] * inv * w[j]);
  }
  for (int j = threadIdx.x + PER * NT; j < hidden; j += NT) o[j] = from_float<T>(x[j] * inv * w[j]);
}

// The same for bfloat16 output and widths that are multiples of 4 up to 16 * NT: 16-byte
// loads, 8-byte stores, the row kept in registers.
template <int NT>
__global__ void __launch_bounds__(NT)
rms_norm_vec_kernel(const float* __restrict__ acc, const float* __restrict__ w, const int* __restrict__ rows,
                    __nv_bfloat16* __restrict__ out, int hidden, float eps) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();

  __shared__ float scratch[32];
  constexpr int PER = 4;  // float4 a thread
  const int r = blockIdx.x;
  const float4* x = reinterpret_cast<const float4*>(acc + (size_t)(rows ? rows[r] : r) * hidden);
  const float4* w4 = reinterpret_cast<const float4*>(w);
  const int quads = hidden >> 2;
  float4 v[PER];
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int j = threadIdx.x + k * NT;
    v[k] = j < quads ? x[j] : make_float4(0.f, 0.f, 0.f, 0.f);
    ss = fmaf(v[k].x, v[k].x, ss);
    ss = fmaf(v[k].y, v[k].y, ss);
    ss = fmaf(v[k].z, v[k].z, ss);
    ss = fmaf(v[k].w, v[k].w, ss);
  }
  ss = block_sum<NT>(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + eps);
  uint2* o = reinterpret_cast<uint2*>(out + (size_t)r * hidden);
#pragma unroll
  for (int k = 0; k < PER; ++k) {
    const int j = threadIdx.x + k * NT;
    if (j < quads) {
      const float4 g = w4[j];
      __nv_bfloat162 lo = __floats2bfloat162_rn(v[k].x * inv * g.x, v[k].y * inv * g.y);
      __nv_bfloat162 hi = __floats2bfloat162_rn(v[k].z * inv * g.z, v[k].w * inv * g.w);
      o[j] = make_uint2(*reinterpret_cast<uint32_t*>(&lo), *reinterpret_cast<uint32_t*>(&hi));
    }
  }
}


// ------------------------------------------------- rotary + cache page write
// qkv: [T, (nh + 2 nkv) d] rows of q heads, k heads, v heads.  For token t at
// position p (angle_i = float(p) * inv_freq[i], split-half pairing i <-> i + d/2):
//   q heads are rotated in place;
//   k heads are rotated and written to the page of (request, p);
//   v heads are copied to the page.
// inv_freq null: nothing is rotated; k and v are copied to the pages as they are.
// Page layout of one cache layer: [page][2 (k, v)][kv head][slot in page][d].
template <typename T>
__global__ void rope_kv_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                               const int* __restrict__ token_req,
                               const int* __restrict__ block_table, int table_width,
                               T* __restrict__ pages, const float* __restrict__ inv_freq, int nh,
                               int nkv, int d, int page_size, int write_kv, int num_pages) {
  tl::pdl_launch_dependents();  // the next kernel may start its prologue (it waits for us before it reads our output)
  tl::pdl_wait();               // everything before us in the stream is complete and visible

  const int t = blockIdx.x;
  const int h = blockIdx.y;
  const int half = d >> 1;
  const int pos = positions[t];
  T* row = qkv + (size_t)t * (nh + 2 * nkv) * d + (size_t)h * d;
  T* dst = row;
  const bool is_v = h >= nh + nkv;
  if (h >= nh) {
    if (!write_kv) return;
    const int kvh = is_v ? h - nh - nkv : h - nh;
    if (!TL_DEBUG_OK(pos >= 0 && pos / page_size < table_width, TL_DEBUG_POSITION, pos)) return;
    const int page = block_table[(size_t)token_req[t] * table_width + pos / page_size];
    if (!TL_DEBUG_OK(page >= 0 && page < num_pages, TL_DEBUG_PAGE, page)) return;
    dst = pages + ((((size_t)page * 2 + (is_v ? 1 : 0)) * nkv + kvh) * page_size + pos % page_size) * d;
  }
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    const float x1 = to_float(row[i]);
    const float x2 = to_float(row[i + half]);
    if (is_v || !inv_freq) {
      if (dst != row) {
        dst[i] = row[i];
        dst[i + half] = row[i + half];
      }
    } else {
      const float angle = (float)pos * inv_freq[i];
      float s, c;
      sincosf(angle, &s, &c);
      dst[i] = from_float<T>(x1 * c - x2 * s);
      dst[i + half] = from_float<T>(x2 * c + x1 * s);
    }
  }
}

// bfloat16, head_dim a multiple of 16: each thread takes 8 consecutive elements of the
// first half of a head and the matching 8 of the second half (two 16-byte loads and
// stores); one block covers several heads of one token.
__global__ void __launch_bounds__(256)
rope_kv_vec_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                   const int* __restrict__ token_req, const int* __restrict__ block_table, int table_width,
                   __nv_bfloat16* __restrict__ pages, const float* __restrict__ inv_freq, int nh, int nkv, int d,
                   int page_size, int heads, int num_pages) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const int t = blockIdx.x;
  const int half = d >> 1;
  const int per_head = half >> 3;  // threads a head
  const int pos = positions[t];
  if (!TL_DEBUG_OK(pos >= 0 && pos / page_size < table_width, TL_DEBUG_POSITION, pos)) return;
  const int page = block_table[(size_t)token_req[t] * table_width + pos / page_size];
  if (!TL_DEBUG_OK(page >= 0 && page < num_pages, TL_DEBUG_PAGE, page)) return;
  const int slot = pos % page_size;
  for (int item = threadIdx.x; item < heads * per_head; item += blockDim.x) {
    const int h = item / per_head, i = (item % per_head) * 8;
    __nv_bfloat16* row = qkv + (size_t)t * (nh + 2 * nkv) * d + (size_t)h * d;
    __nv_bfloat16* dst = row;
    const bool is_v = h >= nh + nkv;
    if (h >= nh) {
      const int kvh = is_v ? h - nh - nkv : h - nh;
      dst = pages + ((((size_t)page * 2 + (is_v ? 1 : 0)) * nkv + kvh) * page_size + slot) * d;
    }
    const uint4 lo = *reinterpret_cast<const uint4*>(row + i);
    const uint4 hi = *reinterpret_cast<const uint4*>(row + i + half);
    if (is_v || !inv_freq) {
      if (dst != row) {
        *reinterpret_cast<uint4*>(dst + i) = lo;
        *reinterpret_cast<uint4*>(dst + i + half) = hi;
      }
      continue;
    }
    float x1[8], x2[8];
    load8(reinterpret_cast<const __nv_bfloat16*>(&lo), x1);
    load8(reinterpret_cast<const __nv_bfloat16*>(&hi), x2);
    uint32_t out_lo[4], out_hi[4];
#pragma unroll
    for (int j = 0; j < 8; j += 2) {
      float s0, c0, s1, c1;
      sincosf((float)pos * inv_freq[i + j], &s0, &c0);
      sincosf((float)pos * inv_freq[i + j + 1], &s1, &c1);
      __nv_bfloat162 a = __floats2bfloat162_rn(x1[j] * c0 - x2[j] * s0, x1[j + 1] * c1 - x2[j + 1] * s1);
      __nv_bfloat162 b = __floats2bfloat162_rn(x2[j] * c0 + x1[j] * s0, x2[j + 1] * c1 + x1[j + 1] * s1);
      out_lo[j >> 1] = *reinterpret_cast<uint32_t*>(&a);
      out_hi[j >> 1] = *reinterpret_cast<uint32_t*>(&b);
    }
    *reinterpret_cast<uint4*>(dst + i) = make_uint4(out_lo[0], out_lo[1], out_lo[2], out_lo[3]);
    *reinterpret_cast<uint4*>(dst + i + half) = make_uint4(out_hi[0], out_hi[1], out_hi[2], out_hi[3]);
  }
}

// ------------------------------------------------------------------- SwiGLU
// out[t, j] = silu(gu[t, j]) * gu[t, I + j],  silu(a) = a * sigmoid(a)
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int inter,
                              size_t total) {
  tl::pdl_launch_dependents();  // the next kernel may start its prologue (it waits for us before it reads our output)
  tl::pdl_wait();               // everything before us in the stream is complete and visible

  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const size_t t = idx / inter;
  const int j = (int)(idx - t * inter);
  const float g = to_float(gu[t * 2 * inter + j]);
  const float u = to_float(gu[t * 2 * inter + inter + j]);
  out[idx] = from_float<T>(g / (1.f + expf(-g)) * u);
}

}  // namespace

TL_DEBUG_READER(tl_elementwise_debug_error)

extern "C" {

int tl_embed(const void* table, int dtype, const int* ids, float* acc, int tokens, int hidden,
             int vocab, cudaStream_t stream) {
  if (tokens <= 0) return 0;
  const int nt = hidden >= 1024 ? 256 : 128;
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(embed_kernel<float>, tokens, nt, 0, stream, (const float*)table, ids, acc, hidden, vocab);
  else
    tl::launch_kernel(embed_kernel<__nv_bfloat16>, tokens, nt, 0, stream, (const __nv_bfloat16*)table, ids, acc, hidden, vocab);
  return TL_LAUNCH_CHECK();
}

int tl_rms_norm(const float* acc, const float* weight, const int* rows, void* out, int out_dtype,
                int num_rows, int hidden, float eps, cudaStream_t stream) {
  if (num_rows <= 0) return 0;
  // the kernel and block size depend on the width, type and alignment alone, so a row's sum
  // never depends on the batch
  const bool aligned = ((reinterpret_cast<uintptr_t>(acc) | reinterpret_cast<uintptr_t>(weight)) & 15) == 0 &&
                       (reinterpret_cast<uintptr_t>(out) & 7) == 0;
  if (out_dtype == TL_DTYPE_BF16 && hidden % 4 == 0 && hidden <= 8192 && aligned) {
    if (hidden <= 2048)
      tl::launch_kernel(rms_norm_vec_kernel<128>, num_rows, 128, 0, stream, acc, weight, rows, (__nv_bfloat16*)out, hidden, eps);
    else if (hidden <= 4096)
      tl::launch_kernel(rms_norm_vec_kernel<256>, num_rows, 256, 0, stream, acc, weight, rows, (__nv_bfloat16*)out, hidden, eps);
    else
      tl::launch_kernel(rms_norm_vec_kernel<512>, num_rows, 512, 0, stream, acc, weight, rows, (__nv_bfloat16*)out, hidden, eps);
    return TL_LAUNCH_CHECK();
  }
  if (hidden <= 2048) {
    if (out_dtype == TL_DTYPE_F32)
      tl::launch_kernel(rms_norm_kernel<float, 256>, num_rows, 256, 0, stream, acc, weight, rows, (float*)out, hidden, eps);
    else
      tl::launch_kernel(rms_norm_kernel<__nv_bfloat16, 256>, num_rows, 256, 0, stream, acc, weight, rows, (__nv_bfloat16*)out, hidden, eps);
  } else {
    if (out_dtype == TL_DTYPE_F32)
      tl::launch_kernel(rms_norm_kernel<float, 512>, num_rows, 512, 0, stream, acc, weight, rows, (float*)out, hidden, eps);
    else
      tl::launch_kernel(rms_norm_kernel<__nv_bfloat16, 512>, num_rows, 512, 0, stream, acc, weight, rows, (__nv_bfloat16*)out, hidden, eps);
  }
  return TL_LAUNCH_CHECK();
}

int tl_rope_kv(void* qkv, int dtype, const int* positions, const int* token_req,
               const int* block_table, int table_width, void* pages, const float* inv_freq,
               int tokens, int nh, int nkv, int d, int page_size, int write_kv, int num_pages,
               cudaStream_t stream) {
  if (tokens <= 0) return 0;
  if (d % 2) return TL_ERR_UNSUPPORTED;
  const int heads = write_kv ? nh + 2 * nkv : nh;
  if (heads > 65535) return TL_ERR_UNSUPPORTED;
  int nt = ((d / 2 + 31) / 32) * 32;
  if (nt > 128) nt = 128;
  if (dtype == TL_DTYPE_BF16 && d % 16 == 0) {
    const int items = heads * (d / 16);
    const int threads = items >= 256 ? 256 : ((items + 31) / 32) * 32;
    tl::launch_kernel(rope_kv_vec_kernel, tokens, threads, 0, stream, (__nv_bfloat16*)qkv, positions, token_req,
                      block_table, table_width, (__nv_bfloat16*)pages, inv_freq, nh, nkv, d, page_size, heads, num_pages);
    return TL_LAUNCH_CHECK();
  }
  dim3 grid(tokens, heads);
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(rope_kv_kernel<float>, grid, nt, 0, stream, (float*)qkv, positions, token_req, block_table,
                                                   table_width, (float*)pages, inv_freq, nh, nkv, d,
                                                   page_size, write_kv, num_pages);
  else
    tl::launch_kernel(rope_kv_kernel<__nv_bfloat16>, grid, nt, 0, stream, 
        (__nv_bfloat16*)qkv, positions, token_req, block_table, table_width, (__nv_bfloat16*)pages,
        inv_freq, nh, nkv, d, page_size, write_kv, num_pages);
  return TL_LAUNCH_CHECK();
}

int tl_swiglu(const void* gate_up, void* out, int dtype, int tokens, int inter,
              cudaStream_t stream) {
  const size_t total = (size_t)tokens * inter;
  if (total == 0) return 0;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  if (dtype == TL_DTYPE_F32)
    tl::launch_kernel(swiglu_kernel<float>, blocks, 256, 0, stream, (const float*)gate_up, (float*)out, inter, total);
  else
    tl::launch_kernel(swiglu_kernel<__nv_bfloat16>, blocks, 256, 0, stream, (const __nv_bfloat16*)gate_up, (__nv_bfloat16*)out, inter, total);
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
