// bfloat16 matrix product on the 5th-generation tensor cores:
//     out[M, N] (+)= x[M, K] . w[N, K]^T (+ bias)          float32 accumulation in TMEM
//
// All kernels share one structure: a producer thread streams 128-byte-swizzled K-major
// tiles of both operands into a ring of shared-memory stages with TMA; one thread issues
// tcgen05.mma (UMMA with 128 or 256 rows, K = 16) from shared-memory descriptors into an
// accumulator in tensor memory and commits each stage back to the producer; four warps
// read the accumulator with tcgen05.ld and run the epilogue (bias -> bf16, accumulate into
// the float32 residual stream, SwiGLU over 16-interleaved gate/up rows, or float32 logits).
//
//   gemm_tc_swapped_kernel     few tokens (decode, M <= 256): the 128 tile rows are WEIGHT
//       rows, so that a handful of tokens still fills the tensor core's M; the tokens are
//       the 16..256 tile columns.  K is split over blockIdx.z and several small CTAs share
//       an SM, so that the weight stream never pauses.  One split writes its output
//       directly; several leave float32 partials [split][M][N] that splitk_finish_kernel
//       (or a fused finishing kernel of the caller) adds in a fixed order.  The weight
//       tiles of the first stages are requested before the wait on the preceding kernel.
//   gemm_tc_persistent_kernel  many tokens: the rows are tokens; one CTA per SM walks over
//       128 x block_q tiles with two accumulators in tensor memory, so that the epilogue of
//       a tile overlaps the next tile's products; block_q is chosen for whole waves.
//   gemm_tc_pair_kernel        the same with pairs of CTAs (cta_group::2) sharing a
//       256 x block_q tile; it runs where its tiles cover no more rows than 128-row tiles would.
//
// Reference counterparts: cuBLAS through nn.Linear (v10_triton_paged_gqa/layer/gqa.py:
// 122-124, 84; model/qwen2_5.py:83-87) and the Triton GEMMs swiglu_kernel/down_kernel
// (v10_triton_paged_gqa/kernel/ffn_swiglu.py:5-164).
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int BLOCK_P = 128;  // tile rows = UMMA M
constexpr int BLOCK_K = 64;   // bf16 per 128-byte row
constexpr int UMMA_K = 16;
constexpr int ROW_TILE_BYTES = BLOCK_P * BLOCK_K * 2;
constexpr int THREADS = 192;

enum Epilogue { EPI_STORE_BF16 = 0, EPI_ACCUM_F32 = 1, EPI_SWIGLU_BF16 = 2, EPI_STORE_F32 = 3 };

__device__ int g_error_word = 0;

struct Params {
  int rows;  // extent of the row operand: tokens (normal) or weight rows (swapped)
  int cols;  // extent of the column operand
  int k_blocks, k_blocks_per_split;
  const float* bias;
  void* out;
  long long ldo;
  int epilogue;
  float* partial;  // [splits][M][N] partial sums (swapped: M = cols, N = rows); nullptr: direct output
  int splits;      // pair kernel: K splits of every tile (1: the tile's epilogue writes the output)
  int ahead;       // stages of weight tiles requested before the wait on the preceding kernel
  // persistent kernel (normal orientation): tile width, stages, tile counts
  int block_q, stages, row_tiles, num_tiles;
};

__device__ __forceinline__ float silu(float g) { return g / (1.f + __expf(-g)); }

// 32 accumulator values of output row m, columns n0 .. n0+31 (normal orientation).
__device__ __forceinline__ void epilogue_chunk(const Params& p, int m, int n0, const float (&v)[32], int cols = 32) {
  const int N = p.cols;
  if (p.epilogue == EPI_SWIGLU_BF16) {
    // columns n0..n0+15 are gate j..j+15, n0+16..n0+31 the matching up values
    if (n0 + 32 > N) return;  // N is a multiple of 32 by construction of the interleave
    __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)m * p.ldo + (n0 >> 1);
    uint32_t packed[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float a = silu(v[2 * j]) * v[2 * j + 16];
      const float b = silu(v[2 * j + 1]) * v[2 * j + 17];
      __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
      packed[j] = *reinterpret_cast<uint32_t*>(&h);
    }
    uint4* dst = reinterpret_cast<uint4*>(o);
    dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
    return;
  }
  if (p.epilogue == EPI_ACCUM_F32 && cols == 32 && n0 + 32 <= N) {
    float* o = (float*)p.out + (size_t)m * p.ldo + n0;
    if ((reinterpret_cast<uintptr_t>(o) & 15) == 0) {
      // all of the chunk's old values are requested before the first is used: one trip to
      // memory a chunk instead of one for every eight columns
      float4* o4 = reinterpret_cast<float4*>(o);
      float4 old[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) old[j] = o4[j];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int n = n0 + 4 * j;
        old[j].x += v[4 * j] + (p.bias ? p.bias[n] : 0.f);
        old[j].y += v[4 * j + 1] + (p.bias ? p.bias[n + 1] : 0.f);
        old[j].z += v[4 * j + 2] + (p.bias ? p.bias[n + 2] : 0.f);
        old[j].w += v[4 * j + 3] + (p.bias ? p.bias[n + 3] : 0.f);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) o4[j] = old[j];
      return;
    }
  }
#pragma unroll
  for (int c = 0; c < 32; c += 8) {
    const int n = n0 + c;
    if (n >= N || c >= cols) return;
    float r[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) r[j] = v[c + j] + ((p.bias && n + j < N) ? p.bias[n + j] : 0.f);
    const bool full = n + 8 <= N;
    if (p.epilogue == EPI_STORE_BF16) {
      __nv_bfloat16* o = (__nv_bfloat16*)p.out + (size_t)m * p.ldo + n;
      if (full && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
        uint32_t packed[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          __nv_bfloat162 h = __floats2bfloat162_rn(r[2 * j], r[2 * j + 1]);
          packed[j] = *reinterpret_cast<uint32_t*>(&h);
        }
        *reinterpret_cast<uint4*>(o) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
      } else {
        for (int j = 0; j < 8 && n + j < N; ++j) o[j] = __float2bfloat16_rn(r[j]);
      }
    } else {
      float* o = (float*)p.out + (size_t)m * p.ldo + n;
      const bool accum = p.epilogue == EPI_ACCUM_F32;
      if (full && ((reinterpret_cast<uintptr_t>(o) & 15) == 0)) {
        float4* o4 = reinterpret_cast<float4*>(o);
        float4 a = make_float4(r[0], r[1], r[2], r[3]), b = make_float4(r[4], r[5], r[6], r[7]);
        if (accum) {
          const float4 x = o4[0], y = o4[1];
          a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
          b.x += y.x; b.y += y.y; b.z += y.z; b.w += y.w;
        }
        o4[0] = a;
        o4[1] = b;
      } else {
        for (int j = 0; j < 8 && n + j < N; ++j) o[j] = accum ? o[j] + r[j] : r[j];
      }
    }
  }
}

// out[row][col0 .. col0 + width) += the accumulator row at ``taddr`` (+ bias), width a multiple of
// 32 and everything 16-byte aligned (the caller checks; warp-uniform).  The old values of a
// chunk are requested one chunk ahead, before the wait for the chunk's tensor-memory read: a
// tile's epilogue is eight dependent trips to memory otherwise, which shows wherever no next
// tile hides it (a CTA's last tile; products of few tiles).  All lanes call it (the tensor-memory
// read is warp-wide); ``live`` lanes touch memory.
__device__ __forceinline__ void accumulate_row(const Params& p, int row, int col0, int width, uint32_t taddr, bool live) {
  float* o = (float*)p.out + (size_t)row * p.ldo + col0;
  float4 cur[8];
  if (live) {
#pragma unroll
    for (int j = 0; j < 8; ++j) cur[j] = reinterpret_cast<const float4*>(o)[j];
  }
#pragma unroll 1
  for (int c = 0; c < width; c += 32) {
    float4 nxt[8];
    const bool more = c + 32 < width;
    if (live && more) {
#pragma unroll
      for (int j = 0; j < 8; ++j) nxt[j] = reinterpret_cast<const float4*>(o + c + 32)[j];
    }
    uint32_t r[32];
    tmem_ld_32(taddr + c, r);
    tmem_ld_wait();
    if (live) {
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int n = col0 + c + 4 * j;
        cur[j].x += __uint_as_float(r[4 * j]) + (p.bias ? p.bias[n] : 0.f);
        cur[j].y += __uint_as_float(r[4 * j + 1]) + (p.bias ? p.bias[n + 1] : 0.f);
        cur[j].z += __uint_as_float(r[4 * j + 2]) + (p.bias ? p.bias[n + 2] : 0.f);
        cur[j].w += __uint_as_float(r[4 * j + 3]) + (p.bias ? p.bias[n + 3] : 0.f);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) reinterpret_cast<float4*>(o + c)[j] = cur[j];
    }
    if (more) {
#pragma unroll
      for (int j = 0; j < 8; ++j) cur[j] = nxt[j];
    }
  }
}

// Whether accumulate_row serves a tile of this width at these columns.
__device__ __forceinline__ bool accumulate_row_serves(const Params& p, int col0, int width) {
  return p.epilogue == EPI_ACCUM_F32 && width % 32 == 0 && col0 + width <= p.cols && p.ldo % 4 == 0 && col0 % 4 == 0 &&
         (reinterpret_cast<uintptr_t>(p.out) & 15) == 0;
}

template <int BLOCK_Q, int STAGES>
__global__ void __launch_bounds__(THREADS)
gemm_tc_swapped_kernel(const __grid_constant__ CUtensorMap map_row, const __grid_constant__ CUtensorMap map_col,
               const Params p) {
  constexpr int COL_TILE_BYTES = BLOCK_Q * BLOCK_K * 2;
  constexpr int STAGE_BYTES = ROW_TILE_BYTES + COL_TILE_BYTES;
  constexpr int TMEM_COLS = BLOCK_Q < 32 ? 32 : BLOCK_Q;
  constexpr uint32_t IDESC = idesc_bf16_f32(BLOCK_P, BLOCK_Q);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty = full + STAGES;
  uint64_t* tmem_full = empty + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = blockIdx.x * BLOCK_P, col0 = blockIdx.y * BLOCK_Q;
  const int kb_begin = blockIdx.z * p.k_blocks_per_split;
  const int kb_end = min(p.k_blocks, kb_begin + p.k_blocks_per_split);
  const int num_kb = kb_end - kb_begin;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(tmem_full, 1);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tensormap(&map_row);
    prefetch_tensormap(&map_col);
  }
  if (warp == 1) {
    tmem_alloc<TMEM_COLS>(tmem_slot);
    tmem_relinquish();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  tl::pdl_launch_dependents();  // the next kernel may start its prologue
  if (warp == 0) {
    if (lane == 0) {
      // Swapped orientation: the row operand is the WEIGHT matrix, which no earlier kernel
      // writes.  Its tiles for the first stages are requested before the wait on the
      // preceding kernel, so the weight stream is already running when the activations
      // (written by that kernel) become available.
      const int ahead = min(min(STAGES, p.ahead), num_kb);
      for (int it = 0; it < ahead; ++it) {
        mbar_expect_tx(&full[it], STAGE_BYTES);
        tma_load_2d(smem + it * STAGE_BYTES, &map_row, &full[it], (kb_begin + it) * BLOCK_K, row0);
      }
      tl::pdl_wait();
      for (int it = 0; it < ahead; ++it)
        tma_load_2d(smem + it * STAGE_BYTES + ROW_TILE_BYTES, &map_col, &full[it], (kb_begin + it) * BLOCK_K, col0);
      for (int it = ahead; it < num_kb; ++it) {
        const int s = it % STAGES;
        const uint32_t phase = (it / STAGES) & 1;
        mbar_wait(&empty[s], phase ^ 1, abort_flag, &g_error_word, 1);
        mbar_expect_tx(&full[s], STAGE_BYTES);
        uint8_t* stage = smem + s * STAGE_BYTES;
        const int k = (kb_begin + it) * BLOCK_K;
        tma_load_2d(stage, &map_row, &full[s], k, row0);
        tma_load_2d(stage + ROW_TILE_BYTES, &map_col, &full[s], k, col0);
      }
    } else {
      tl::pdl_wait();
    }
  } else if (warp == 1) {
    tl::pdl_wait();
    // The whole warp walks the loop and waits; one elected lane issues (see the persistent kernel)
    const uint64_t a_desc0 = smem_desc_sw128(smem_addr(smem));
    const uint64_t b_desc0 = smem_desc_sw128(smem_addr(smem + ROW_TILE_BYTES));
    int s = 0;
    uint32_t phase = 0;
    for (int it = 0; it < num_kb; ++it) {
      mbar_wait(&full[s], phase, abort_flag, &g_error_word, 2);
      fence_after_sync();
      const uint64_t a_desc = a_desc0 + (uint64_t)(s * (STAGE_BYTES >> 4));
      const uint64_t b_desc = b_desc0 + (uint64_t)(s * (STAGE_BYTES >> 4));
      if (elect_one()) {
#pragma unroll
        for (int k = 0; k < BLOCK_K / UMMA_K; ++k) {
          // 16 bf16 = 32 bytes further along K inside the swizzled row: +2 in 16-byte units
          mma_bf16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, IDESC, it > 0 || k > 0);
        }
        mma_commit(&empty[s]);
        if (it == num_kb - 1) mma_commit(tmem_full);
      }
      __syncwarp();
      if (++s == STAGES) {
        s = 0;
        phase ^= 1;
      }
    }
    if (num_kb == 0 && elect_one()) mma_commit(tmem_full);
    __syncwarp();
  } else {
    tl::pdl_wait();  // the epilogue writes buffers that earlier kernels may still read
    mbar_wait(tmem_full, 0, abort_flag, &g_error_word, 3);
    fence_after_sync();
    const int quarter = warp & 3;  // the TMEM lane quarter this warp may read
    const int row = row0 + quarter * 32 + lane;
    const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
    constexpr int CHUNK = BLOCK_Q < 32 ? 16 : 32;
#pragma unroll 1
    for (int c = 0; c < BLOCK_Q; c += CHUNK) {
      float v[32];
      if constexpr (CHUNK == 32) {
        uint32_t r[32];
        tmem_ld_32(taddr + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
      } else {
        uint32_t r[16];
        tmem_ld_16(taddr + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
#pragma unroll
        for (int j = 16; j < 32; ++j) v[j] = 0.f;
      }
      const bool live = row < p.rows && num_kb > 0;
      // row = weight row n, columns = tokens m
      if (p.partial != nullptr) {  // partial[split][m][n]; the finishing kernel adds the splits
        if (live) {
          float* dst = p.partial + ((size_t)blockIdx.z * p.cols) * p.rows + row;
#pragma unroll
          for (int j = 0; j < CHUNK; ++j) {
            const int m = col0 + c + j;
            if (m < p.cols) dst[(size_t)m * p.rows] = v[j];
          }
        }
      } else if (p.epilogue == EPI_SWIGLU_BF16) {
        // lanes 0-15 hold gate rows, lanes 16-31 the matching up rows (interleave of 16)
        const int out_col = ((row0 + quarter * 32) >> 1) + lane;
#pragma unroll
        for (int j = 0; j < CHUNK; ++j) {
          const float up = __shfl_down_sync(0xffffffffu, v[j], 16);
          const int m = col0 + c + j;
          if (live && lane < 16 && m < p.cols)
            ((__nv_bfloat16*)p.out)[(size_t)m * p.ldo + out_col] = __float2bfloat16_rn(silu(v[j]) * up);
        }
      } else if (live) {
        const float b = p.bias ? p.bias[row] : 0.f;
#pragma unroll
        for (int j = 0; j < CHUNK; ++j) {
          const int m = col0 + c + j;
          if (m >= p.cols) break;
          const float r = v[j] + b;
          if (p.epilogue == EPI_STORE_BF16)
            ((__nv_bfloat16*)p.out)[(size_t)m * p.ldo + row] = __float2bfloat16_rn(r);
          else if (p.epilogue == EPI_ACCUM_F32)
            ((float*)p.out)[(size_t)m * p.ldo + row] += r;
          else
            ((float*)p.out)[(size_t)m * p.ldo + row] = r;
        }
      }
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc<TMEM_COLS>(tmem_base);
  }
}

// Normal orientation, persistent: one CTA per SM walks over output tiles (row tiles
// fastest, so CTAs running at the same time share weight tiles in L2).  The tile width
// block_q (a multiple of 16 up to 256) is chosen on the host so that the tiles fill whole
// waves.  The accumulator is double-buffered in tensor memory (2 x 256 columns): while the
// four epilogue warps drain tile i, the MMA thread already accumulates tile i + 1, and the
// TMA producer never stops between tiles.
__global__ void __launch_bounds__(THREADS, 1)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap map_row, const __grid_constant__ CUtensorMap map_col,
                          const Params p) {
  constexpr int MAX_STAGES = 8;
  constexpr int ACC_COLS = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int stage_bytes = ROW_TILE_BYTES + p.block_q * BLOCK_K * 2;
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.stages * stage_bytes);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* tmem_full = empty + MAX_STAGES;   // [2]
  uint64_t* tmem_empty = tmem_full + 2;        // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 4);  // one arrival from each epilogue warp
    }
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tensormap(&map_row);
    prefetch_tensormap(&map_col);
  }
  if (warp == 1) {
    tmem_alloc<512>(tmem_slot);
    tmem_relinquish();
  }
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  tl::pdl_launch_dependents();
  tl::pdl_wait();  // activations come from the preceding kernel

  const int num_kb = p.k_blocks;
  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x) {
        const int row0 = (tile % p.row_tiles) * BLOCK_P, col0 = (tile / p.row_tiles) * p.block_q;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(&empty[s], phase ^ 1, abort_flag, &g_error_word, 1);
          mbar_expect_tx(&full[s], stage_bytes);
          uint8_t* stage = smem + s * stage_bytes;
          tma_load_2d(stage, &map_row, &full[s], kb * BLOCK_K, row0);
          tma_load_2d(stage + ROW_TILE_BYTES, &map_col, &full[s], kb * BLOCK_K, col0);
          if (++s == p.stages) {
            s = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // The whole warp walks the loop and waits; one elected lane issues.  (Inside a one-lane
    // branch the operands of every MMA go through per-lane registers, which makes the issue
    // slower; the tensor core's queue is short, so what this warp spends between two MMAs
    // shows.)
    const uint32_t idesc = idesc_bf16_f32(BLOCK_P, p.block_q);
    const uint64_t a_desc0 = smem_desc_sw128(smem_addr(smem));
    const uint64_t b_desc0 = smem_desc_sw128(smem_addr(smem + ROW_TILE_BYTES));
    const uint64_t stage_step = (uint64_t)(stage_bytes >> 4);  // in the descriptors' address field
    int s = 0, local = 0;
    uint32_t phase = 0;
    uint64_t a_desc = a_desc0, b_desc = b_desc0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++local) {
      const int a = local & 1;
      mbar_wait(&tmem_empty[a], ((local >> 1) & 1) ^ 1, abort_flag, &g_error_word, 4);
      const uint32_t acc = tmem_base + a * ACC_COLS;
      for (int kb = 0; kb < num_kb; ++kb) {
        mbar_wait(&full[s], phase, abort_flag, &g_error_word, 2);
        fence_after_sync();
        if (elect_one()) {
#pragma unroll
          for (int k = 0; k < BLOCK_K / UMMA_K; ++k) mma_bf16(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, kb > 0 || k > 0);
          mma_commit(&empty[s]);
          if (kb == num_kb - 1) mma_commit(&tmem_full[a]);
        }
        __syncwarp();
        a_desc += stage_step;
        b_desc += stage_step;
        if (++s == p.stages) {
          s = 0;
          phase ^= 1;
          a_desc = a_desc0;
          b_desc = b_desc0;
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    int local = 0;
    for (int tile = blockIdx.x; tile < p.num_tiles; tile += gridDim.x, ++local) {
      const int a = local & 1;
      const int row0 = (tile % p.row_tiles) * BLOCK_P, col0 = (tile / p.row_tiles) * p.block_q;
      mbar_wait(&tmem_full[a], (local >> 1) & 1, abort_flag, &g_error_word, 3);
      fence_after_sync();
      const int row = row0 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + a * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
      const bool live = row < p.rows;
      const bool whole = accumulate_row_serves(p, col0, p.block_q);
      if (whole) accumulate_row(p, row, col0, p.block_q, taddr, live);
#pragma unroll 1
      for (int c = whole ? p.block_q : 0; c < p.block_q; c += 32) {
        float v[32];
        const int cols = min(32, p.block_q - c);
        if (cols == 32) {
          uint32_t r[32];
          tmem_ld_32(taddr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        } else {
          uint32_t r[16];
          tmem_ld_16(taddr + c, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __uint_as_float(r[j]);
#pragma unroll
          for (int j = 16; j < 32; ++j) v[j] = 0.f;
        }
        if (live) epilogue_chunk(p, row, col0 + c, v, cols);
      }
      // the accumulator may be overwritten once all four warps have read it
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty[a]);
    }
  }
  fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc<512>(tmem_base);
  }
}

// Normal orientation, persistent, CTA PAIRS (cta_group::2): a cluster of two CTAs on
// neighbouring SMs computes a 256 x block_q tile.  CTA r of the pair loads rows
// [128 r, 128 r + 128) of the A tile and columns [r block_q / 2, (r + 1) block_q / 2) of the
// B tile into its own shared memory; one thread of CTA 0 issues tcgen05.mma.cta_group::2
// (UMMA 256 x block_q x 16), which reads both CTAs' shared memory and writes 128
// accumulator rows into each CTA's tensor memory.  Against the single-CTA kernel each SM
// moves a third less data into shared memory per flop (32 KB instead of 48 KB per k-block
// at block_q = 256), which is what bounds that kernel, and has 6 stages instead of 4.
// Barriers: the TMA loads of both CTAs count on CTA 0's "full" barrier; tcgen05.commit
// arrives on the "empty" and "accumulator full" barriers of both CTAs; the epilogue warps
// of both CTAs arrive on CTA 0's "accumulator empty" barrier.
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(THREADS, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap map_row, const __grid_constant__ CUtensorMap map_col,
                    const Params p) {
  constexpr int MAX_STAGES = 8;
  constexpr int ACC_COLS = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const int half_q = p.block_q / 2;
  const int stage_bytes = ROW_TILE_BYTES + half_q * BLOCK_K * 2;  // of ONE CTA
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + p.stages * stage_bytes);
  uint64_t* empty = full + MAX_STAGES;
  uint64_t* tmem_full = empty + MAX_STAGES;  // [2]
  uint64_t* tmem_empty = tmem_full + 2;       // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t rank = cluster_rank();
  const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tmem_full[a], 1);
      mbar_init(&tmem_empty[a], 8);  // four epilogue warps in each CTA of the pair
    }
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tensormap(&map_row);
    prefetch_tensormap(&map_col);
  }
  if (warp == 1) {
    tmem_alloc_pair<512>(tmem_slot);
    tmem_relinquish_pair();
  }
  fence_before_sync();
  cluster_sync();  // barriers of both CTAs are initialised before anyone signals them
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  tl::pdl_launch_dependents();
  tl::pdl_wait();

  // A work item is one K split of one tile; the splits of a tile are num_tiles items apart
  const int num_items = p.num_tiles * p.splits;
  if (warp == 0) {
    if (lane == 0) {
      int s = 0;
      uint32_t phase = 0;
      for (int item = pair; item < num_items; item += num_pairs) {
        const int tile = item % p.num_tiles, kb0 = (item / p.num_tiles) * p.k_blocks_per_split;
        const int kb1 = min(p.k_blocks, kb0 + p.k_blocks_per_split);
        const int row0 = (tile % p.row_tiles) * 256 + (int)rank * BLOCK_P;
        const int col0 = (tile / p.row_tiles) * p.block_q + (int)rank * half_q;
        for (int kb = kb0; kb < kb1; ++kb) {
          mbar_wait(&empty[s], phase ^ 1, abort_flag, &g_error_word, 1);
          if (rank == 0) mbar_expect_tx(&full[s], 2 * stage_bytes);  // the bytes of both CTAs
          const uint32_t bar = peer_addr(&full[s], 0);
          uint8_t* stage = smem + s * stage_bytes;
          tma_load_2d_pair(stage, &map_row, bar, kb * BLOCK_K, row0);
          tma_load_2d_pair(stage + ROW_TILE_BYTES, &map_col, bar, kb * BLOCK_K, col0);
          if (++s == p.stages) {
            s = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0) {  // the whole warp walks the loop and waits; one elected lane issues
      const uint32_t idesc = idesc_bf16_f32(256, p.block_q);
      const uint64_t a_desc0 = smem_desc_sw128(smem_addr(smem));
      const uint64_t b_desc0 = smem_desc_sw128(smem_addr(smem + ROW_TILE_BYTES));
      const uint64_t stage_step = (uint64_t)(stage_bytes >> 4);  // in the descriptors' address field
      int s = 0, local = 0;
      uint32_t phase = 0;
      uint64_t a_desc = a_desc0, b_desc = b_desc0;
      for (int item = pair; item < num_items; item += num_pairs, ++local) {
        const int a = local & 1;
        const int kb0 = (item / p.num_tiles) * p.k_blocks_per_split;
        const int num_kb = min(p.k_blocks, kb0 + p.k_blocks_per_split) - kb0;
        mbar_wait(&tmem_empty[a], ((local >> 1) & 1) ^ 1, abort_flag, &g_error_word, 4);
        const uint32_t acc = tmem_base + a * ACC_COLS;
        for (int kb = 0; kb < num_kb; ++kb) {
          mbar_wait(&full[s], phase, abort_flag, &g_error_word, 2);
          fence_after_sync();
          if (elect_one()) {
#pragma unroll
            for (int k = 0; k < BLOCK_K / UMMA_K; ++k)
              mma_bf16_pair(acc, a_desc + 2 * k, b_desc + 2 * k, idesc, kb > 0 || k > 0);
            mma_commit_pair(&empty[s]);
            if (kb == num_kb - 1) mma_commit_pair(&tmem_full[a]);
          }
          __syncwarp();
          a_desc += stage_step;
          b_desc += stage_step;
          if (++s == p.stages) {
            s = 0;
            phase ^= 1;
            a_desc = a_desc0;
            b_desc = b_desc0;
          }
        }
      }
    }
  } else {
    const int quarter = warp & 3;
    int local = 0;
    Params e = p;  // where and how an item's values go: with K splits, as float32 into the split's plane
    if (p.partial != nullptr) {
      e.epilogue = EPI_STORE_F32;
      e.bias = nullptr;
      e.ldo = p.cols;
    }
    for (int item = pair; item < num_items; item += num_pairs, ++local) {
      const int a = local & 1;
      const int tile = item % p.num_tiles;
      const int row0 = (tile % p.row_tiles) * 256 + (int)rank * BLOCK_P, col0 = (tile / p.row_tiles) * p.block_q;
      if (p.partial != nullptr) e.out = p.partial + (size_t)(item / p.num_tiles) * p.rows * p.cols;
      mbar_wait(&tmem_full[a], (local >> 1) & 1, abort_flag, &g_error_word, 3);
      fence_after_sync();
      const int row = row0 + quarter * 32 + lane;
      const uint32_t taddr = tmem_base + a * ACC_COLS + ((uint32_t)(quarter * 32) << 16);
      const bool live = row < p.rows;
      const bool whole = accumulate_row_serves(e, col0, p.block_q);
      if (whole) accumulate_row(e, row, col0, p.block_q, taddr, live);
#pragma unroll 1
      for (int c = whole ? p.block_q : 0; c < p.block_q; c += 32) {
        float v[32];
        uint32_t r[32];
        tmem_ld_32(taddr + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
        if (live) epilogue_chunk(e, row, col0 + c, v, 32);
      }
      fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(peer_addr(&tmem_empty[a], 0));
    }
  }
  __syncwarp();
  fence_before_sync();
  cluster_sync();  // neither CTA leaves while its peer may still read its memory or signal it
  if (warp == 1) {
    fence_after_sync();
    tmem_dealloc_pair<512>(tmem_base);
  }
}

// Adds the split partials [splits][M][N] in ascending split order and applies the epilogue.
__global__ void splitk_finish_kernel(const float* __restrict__ partial, int splits, int M, int N,
                                     const float* __restrict__ bias, int epilogue, void* out, long long ldo) {
  tl::pdl_wait();               // everything before us in the stream is complete and visible
  tl::pdl_launch_dependents();  // the next kernel may start its own prologue

  const int out_cols = epilogue == EPI_SWIGLU_BF16 ? N / 2 : N;
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (long long)M * out_cols) return;
  const int m = (int)(idx / out_cols), c = (int)(idx % out_cols);
  const size_t plane = (size_t)M * N;
  if (epilogue == EPI_SWIGLU_BF16) {
    const int g = (c >> 4) * 32 + (c & 15);
    float gate = 0.f, up = 0.f;
    for (int s = 0; s < splits; ++s) {
      gate += partial[s * plane + (size_t)m * N + g];
      up += partial[s * plane + (size_t)m * N + g + 16];
    }
    ((__nv_bfloat16*)out)[(size_t)m * ldo + c] = __float2bfloat16_rn(silu(gate) * up);
    return;
  }
  float v = 0.f;
  for (int s = 0; s < splits; ++s) v += partial[s * plane + (size_t)m * N + c];
  if (bias) v += bias[c];
  if (epilogue == EPI_STORE_BF16)
    ((__nv_bfloat16*)out)[(size_t)m * ldo + c] = __float2bfloat16_rn(v);
  else if (epilogue == EPI_ACCUM_F32)
    ((float*)out)[(size_t)m * ldo + c] += v;
  else
    ((float*)out)[(size_t)m * ldo + c] = v;
}

// ------------------------------------------------------------------ host side
struct MapKey {
  const void* base;
  uint64_t rows, cols, ld;
  uint32_t box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && ld == o.ld && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.base);
    h = h * 1000003u ^ k.rows;
    h = h * 1000003u ^ k.cols;
    h = h * 1000003u ^ k.ld;
    return h * 1000003u ^ k.box_rows;
  }
};

bool cached_map(CUtensorMap* out, const void* base, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_rows) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex lock;
  const MapKey key{base, rows, cols, ld, box_rows};
  std::lock_guard<std::mutex> guard(lock);
  auto it = cache.find(key);
  if (it == cache.end()) {
    CUtensorMap map;
    if (!tc_host::make_map_bf16(&map, base, rows, cols, ld, box_rows)) return false;
    if (cache.size() > 4096) cache.clear();
    it = cache.emplace(key, map).first;
  }
  *out = it->second;
  return true;
}

int sm_count() {
  static int count = 0;
  if (!count) {
    int device = 0;
    cudaGetDevice(&device);
    cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, device);
    if (count <= 0) count = 148;
  }
  return count;
}

// The swapped orientation is considered up to this many tokens (TORCHLET_B200_SWAP_MAX forces
// another bound, for measurements).
int swap_max_tokens() {
  static int value = -1;
  if (value < 0) {
    const char* v = getenv("TORCHLET_B200_SWAP_MAX");
    value = v ? atoi(v) : 256;
    if (value < 0 || value > 256) value = 256;
  }
  return value;
}

int pick_block_q_swapped(int M) {
  if (M <= 16) return 16;
  if (M <= 32) return 32;
  if (M <= 64) return 64;
  if (M <= 128) return 128;
  return 256;
}

struct Plan {
  bool swap;   // swapped orientation (rows = weight rows)
  bool pairs;  // normal orientation: the CTA-pair kernel
  int block_q, splits, k_blocks_per_split;
};

// The tile width that gives the shortest schedule of the persistent kernels, and its cost:
// waves of one tile per SM (per SM pair), a tile's time in proportion to its width plus a
// fixed part.  Single CTAs take 128 rows and widths 64..256 in steps of 16, pairs 256 rows and
// widths 128..256 in steps of 32.
long long best_width(int M, int N, bool pairs, int* width) {
  const int units = pairs ? sm_count() / 2 : sm_count();
  const int row_tiles = (M + (pairs ? 255 : BLOCK_P - 1)) / (pairs ? 256 : BLOCK_P);
  long long best_cost = -1;
  for (int q = 256; q >= (pairs ? 128 : 64); q -= (pairs ? 32 : 16)) {
    const long long tiles = (long long)row_tiles * ((N + q - 1) / q);
    const long long cost = ((tiles + units - 1) / units) * (q + 24);
    if (best_cost < 0 || cost < best_cost) {
      best_cost = cost;
      *width = q;
    }
  }
  return best_cost;
}

// K splits of the CTA-pair kernel for ONE row tile (129-256 tokens) times a narrow output and a
// long K, like the down projection: 14 tiles of width 256 leave 60 of 74 SM pairs idle, and one
// pair needs 100 us for K = 18,944.  Measured on that product at 256 tokens: 100 / 67 / 57 / 50 /
// 51 us with 1 / 2 / 3 / 4 / 5 splits (the swapped kernel: 63 us).  With two row tiles (512
// tokens) or K = 3,584 no split count gained anything: all SMs together take in operands at
// 8-10 TB/s from the L2, which is what those sizes run into either way.
bool pair_split_plan(int M, int N, int K, int* width, int* splits_out, int* k_blocks_per_split) {
  const int k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
  const int tiles = (N + 255) / 256, pairs = sm_count() / 2;
  if (M > 256 || k_blocks < 128 || 2 * tiles > pairs) return false;
  int splits = pairs / tiles;
  if (splits > 4) splits = 4;
  *width = 256;
  *k_blocks_per_split = (k_blocks + splits - 1) / splits;
  *splits_out = (k_blocks + *k_blocks_per_split - 1) / *k_blocks_per_split;
  return true;
}

// TORCHLET_B200_PAIR_SPLITS=0 switches the K splits of the pair kernel off (for measurements).
bool pair_splits_enabled() {
  static int value = -1;
  if (value < 0) {
    const char* v = getenv("TORCHLET_B200_PAIR_SPLITS");
    value = (v && atoi(v) == 0) ? 0 : 1;
  }
  return value == 1;
}

Plan make_plan(int M, int N, int K) {
  Plan plan;
  const int k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
  // In the normal orientation the CTA-pair kernel runs where its 256-row tiles cover no more rows
  // than 128-row tiles would (129-256, 385-512, ... tokens) and from 1,024 tokens on
  const bool pair_rows = sm_count() % 2 == 0 && (M >= 1024 || (M + 255) / 256 * 256 == (M + BLOCK_P - 1) / BLOCK_P * BLOCK_P);
  int pair_q = 256, pair_n = 1, pair_kb = k_blocks;
  best_width(M, N, true, &pair_q);
  const bool pair_splits = pair_rows && pair_splits_enabled() && pair_split_plan(M, N, K, &pair_q, &pair_n, &pair_kb);
  // Which orientation.  Up to 64 tokens the swapped kernel streams the weights at 5.5-6.2 TB/s.
  // Beyond that its wide column tiles lose (4.7 TB/s at 128 columns, 2.5 at 256), and the
  // persistent kernels take over where they have a tile for every SM, or, past 128 tokens, where
  // one CTA's pass over K (about 200 GB/s a CTA) is shorter than the swapped kernel's time or
  // the pair kernel splits K.
  plan.swap = M <= swap_max_tokens();
  if (plan.swap && M > 64 && swap_max_tokens() == 256) {
    const long long normal_tiles = (long long)((M + BLOCK_P - 1) / BLOCK_P) * ((N + 255) / 256);
    const double pass_us = (double)K * (BLOCK_P + 256) * 2 / 200e3;
    const double swapped_us = (double)N * K * 2 / 2.5e6 + 8.0;
    if (normal_tiles >= sm_count() || (M > 128 && (pass_us < swapped_us || pair_splits)))
      plan.swap = false;
  }
  // Up to 256 tokens the pair kernel needs a tile for every pair (the gate/up product, the LM head)
  // or its K splits; the o and qkv products are a little faster in the single-CTA kernel there
  // (256 tokens: 20 against 23 us)
  plan.pairs = !plan.swap && pair_rows &&
               (M > 256 || pair_splits || (long long)((N + 255) / 256) >= sm_count() / 2);
  if (plan.swap) {
    plan.block_q = pick_block_q_swapped(M);
    const int tiles = ((N + BLOCK_P - 1) / BLOCK_P) * ((M + plan.block_q - 1) / plan.block_q);
    const int ctas_per_sm = plan.block_q <= 128 ? 2 : 1;
    int splits = ctas_per_sm * sm_count() / tiles;
    // few tiles (the qkv, o and down products): three quarters of that; fewer, longer splits
    // leave the finishing kernel less to add (measured: -1.2 % of a batch-8 decode step; six stages
    // and two CTAs an SM for the 16-token tile instead of four and three: another -0.9 %)
    if (tiles < 100) splits = splits * 3 / 4;
    if (splits < 1) splits = 1;
    if (splits > k_blocks / 4) splits = k_blocks / 4 > 0 ? k_blocks / 4 : 1;  // at least 4 k-blocks a split
    plan.k_blocks_per_split = (k_blocks + splits - 1) / splits;
    plan.splits = (k_blocks + plan.k_blocks_per_split - 1) / plan.k_blocks_per_split;
  } else if (plan.pairs) {
    plan.block_q = pair_q;
    plan.splits = pair_n;
    plan.k_blocks_per_split = pair_kb;
  } else {
    best_width(M, N, false, &plan.block_q);
    plan.splits = 1;
    plan.k_blocks_per_split = k_blocks;
  }
  return plan;
}

template <int BLOCK_Q, int STAGES>
int launch_swapped(const CUtensorMap& map_row, const CUtensorMap& map_col, const Params& p, dim3 grid, cudaStream_t stream) {
  constexpr int SMEM = STAGES * (ROW_TILE_BYTES + BLOCK_Q * BLOCK_K * 2) + 1024 + 256;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(gemm_tc_swapped_kernel<BLOCK_Q, STAGES>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  tl::launch_kernel(gemm_tc_swapped_kernel<BLOCK_Q, STAGES>, grid, THREADS, SMEM, stream, map_row, map_col, p);
  return TL_LAUNCH_CHECK();
}

// A wait that nothing ends, with a limit of 2^16 cycles (tens of microseconds): the same
// mbar_wait the products use gives up, leaves its code in the error word and in the block's
// abort flag, the block's second wait then gives up at once, and the kernel returns normally.
__global__ void wait_selftest_kernel(int code) {
  tl::pdl_wait();
  tl::pdl_launch_dependents();
  __shared__ uint64_t bar;
  __shared__ int abort_word;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_word = 0;
    mbar_fence_init();
  }
  __syncthreads();
  volatile int* abort_flag = &abort_word;
  if (threadIdx.x == 0) {
    mbar_wait(&bar, 0, abort_flag, &g_error_word, code, 1ll << 16);  // nobody arrives
    mbar_wait(&bar, 0, abort_flag, &g_error_word, code + 1);         // the block has given up: a short limit
  }
  __syncthreads();
}

}  // namespace

extern "C" {

// Shows, without a fault or a hang, what happens when a bounded wait runs out: launches one
// block that waits on a barrier nobody arrives at (limit 2^16 cycles).  Afterwards
// tl_gemm_tc_error() returns ``code``.  For tests of the error path.
int tl_gemm_tc_wait_selftest(int code, cudaStream_t stream) {
  if (code <= 0) return TL_ERR_UNSUPPORTED;
  tl::launch_kernel(wait_selftest_kernel, 1, 32, 0, stream, code);
  return TL_LAUNCH_CHECK();
}

// How a product of these sizes would run: *swap (0/1), *splits; returns the bytes of
// float32 workspace it needs (partial sums: the swapped orientation, K splits of the pair kernel).
long long tl_gemm_tc_plan(int M, int N, int K, int* swap, int* splits) {
  const Plan plan = make_plan(M, N, K);
  if (swap) *swap = plan.swap ? 1 : 0;
  if (splits) *splits = plan.splits;
  return (plan.swap || plan.splits > 1) ? (long long)plan.splits * M * N * 4 : 0;
}

// Reads and clears the error word that a bounded wait sets when it gives up.
int tl_gemm_tc_error() {
  int value = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&value, g_error_word, sizeof(int)) != cudaSuccess) return -1;
  if (value) cudaMemcpyToSymbol(g_error_word, &zero, sizeof(int));
  return value;
}

// defer == 1 (products that run with partial sums: *splits of tl_gemm_tc_plan > 1, or swapped):
// leave the float32 partials [splits][M][N] in the workspace for a fused finishing kernel of the
// caller; *splits_out gets their number.
// In the normal orientation the CTA-pair kernel (cta_group::2) runs where its 256-row tiles cover
// no more rows than 128-row tiles would (129-256, 385-512, ... tokens) and from 1,024 tokens on;
// measured faster there on every product of the model, by 3-14 %: 1,585 against 1,445 TFLOP/s on
// the gate/up product at 2,048 tokens, 100 against 115 us at 448, 60 against 69 us at 200; slower
// by 1-7 % at 272 and 384.  The single-CTA persistent kernel takes the rest; defer == 2 forces
// the pair kernel, defer == 3 the single-CTA kernel (both without K splits).
// out (+)= x[M, K] . w[N, K]^T.  x and w bfloat16 with K contiguous, ldx/ldw elements
// between rows (multiples of 8, bases 16-byte aligned).  epilogue: 0 bf16 out + bias,
// 1 float32 out += result, 2 SwiGLU over 16-interleaved gate/up rows of w -> bf16
// [M, N/2], 3 float32 out.  workspace: float32 scratch of at least tl_gemm_tc_plan bytes.
int tl_gemm_tc(const void* x, const void* w, const float* bias, void* out, long long ldo, int epilogue, int M,
               int N, int K, long long ldx, long long ldw, void* workspace, long long workspace_bytes, int defer,
               int* splits_out, cudaStream_t stream) {
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || K % 8 || ldx % 8 || ldw % 8 || epilogue < 0 || epilogue > 3) return TL_ERR_UNSUPPORTED;
  if (epilogue == EPI_SWIGLU_BF16 && (N % 32 || bias)) return TL_ERR_UNSUPPORTED;
  const Plan plan = make_plan(M, N, K);
  Params p;
  p.k_blocks = (K + BLOCK_K - 1) / BLOCK_K;
  p.k_blocks_per_split = plan.k_blocks_per_split;
  p.bias = bias;
  p.out = out;
  p.ldo = ldo;
  p.epilogue = epilogue;
  p.partial = nullptr;
  p.splits = 1;
  p.ahead = 8;  // all stages
  if (splits_out) *splits_out = 0;
  CUtensorMap map_row, map_col;
  int rc;
  const bool pair_splits = !plan.swap && plan.pairs && plan.splits > 1 && defer <= 1;
  if (!plan.swap && defer == 1 && !pair_splits) return TL_ERR_UNSUPPORTED;
  if (plan.swap && defer >= 2) defer = 0;
  const bool pairs = !plan.swap && sm_count() % 2 == 0 && (defer == 2 || (defer <= 1 && plan.pairs));
  if (plan.swap) {
    // one split writes its output directly; several (or a deferred finish) go through partials
    const bool partials = plan.splits > 1 || defer;
    if (partials) {
      if ((long long)plan.splits * M * N * 4 > workspace_bytes) return TL_ERR_UNSUPPORTED;
      p.partial = (float*)workspace;
    }
    p.rows = N;
    p.cols = M;
    if (!cached_map(&map_row, w, N, K, ldw, BLOCK_P) || !cached_map(&map_col, x, M, K, ldx, plan.block_q))
      return TL_ERR_UNSUPPORTED;
    dim3 grid((N + BLOCK_P - 1) / BLOCK_P, (M + plan.block_q - 1) / plan.block_q, plan.splits);
    switch (plan.block_q) {
      // few stages a CTA, several CTAs an SM: while one CTA starts up or runs its epilogue
      // the others keep the weight stream going
      case 16: rc = launch_swapped<16, 6>(map_row, map_col, p, grid, stream); break;    // 108 KB: 2 CTAs/SM
      case 32: rc = launch_swapped<32, 4>(map_row, map_col, p, grid, stream); break;    //  80 KB: 2 CTAs/SM
      case 64: rc = launch_swapped<64, 4>(map_row, map_col, p, grid, stream); break;    //  96 KB: 2 CTAs/SM
      case 128: rc = launch_swapped<128, 3>(map_row, map_col, p, grid, stream); break;  //  96 KB: 2 CTAs/SM
      default: rc = launch_swapped<256, 4>(map_row, map_col, p, grid, stream); break;
    }
    if (rc || !partials) return rc;
    if (defer) {
      if (splits_out) *splits_out = plan.splits;
      return 0;
    }
    const int out_cols = epilogue == EPI_SWIGLU_BF16 ? N / 2 : N;
    const long long total = (long long)M * out_cols;
    tl::launch_kernel(splitk_finish_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, p.partial, plan.splits, M, N, bias,
                                                                             epilogue, out, ldo);
    return TL_LAUNCH_CHECK();
  }
  p.rows = M;
  p.cols = N;
  constexpr int SMEM_LIMIT = 227 * 1024;
  if (pairs) {
    // CTA pairs: 256-row tiles, tile width a multiple of 32 chosen for whole waves of pairs
    const int num_pairs = sm_count() / 2;
    const int row_tiles = (M + 255) / 256;
    int block_q = 256;
    if (plan.pairs && defer <= 1)
      block_q = plan.block_q;
    else
      best_width(M, N, true, &block_q);
    if (pair_splits) {  // partial sums [splits][M][N], added by the finishing pass below or by the caller's
      if ((long long)plan.splits * M * N * 4 > workspace_bytes) return TL_ERR_UNSUPPORTED;
      p.partial = (float*)workspace;
      p.splits = plan.splits;
    } else {
      p.k_blocks_per_split = p.k_blocks;
    }
    if (!cached_map(&map_row, x, M, K, ldx, BLOCK_P) || !cached_map(&map_col, w, N, K, ldw, block_q / 2))
      return TL_ERR_UNSUPPORTED;
    p.block_q = block_q;
    p.row_tiles = row_tiles;
    p.num_tiles = row_tiles * ((N + block_q - 1) / block_q);
    const int stage_bytes = ROW_TILE_BYTES + (block_q / 2) * BLOCK_K * 2;
    p.stages = (SMEM_LIMIT - 1024 - 512) / stage_bytes;
    if (p.stages > 8) p.stages = 8;
    const int smem = p.stages * stage_bytes + 1024 + 512;
    static bool configured = false;
    if (!configured) {
      cudaError_t err = cudaFuncSetAttribute(gemm_tc_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             SMEM_LIMIT);
      if (err != cudaSuccess) return (int)err;
      configured = true;
    }
    const int items = p.num_tiles * p.splits;
    const int ctas = 2 * (items < num_pairs ? items : num_pairs);
    tl::launch_kernel(gemm_tc_pair_kernel, dim3(ctas), THREADS, smem, stream, map_row, map_col, p);
    rc = TL_LAUNCH_CHECK();
    if (rc || !pair_splits) return rc;
    if (defer == 1) {
      if (splits_out) *splits_out = plan.splits;
      return 0;
    }
    const int out_cols = epilogue == EPI_SWIGLU_BF16 ? N / 2 : N;
    const long long total = (long long)M * out_cols;
    tl::launch_kernel(splitk_finish_kernel, (unsigned)((total + 255) / 256), 256, 0, stream, p.partial, plan.splits, M, N,
                      bias, epilogue, out, ldo);
    return TL_LAUNCH_CHECK();
  }
  p.k_blocks_per_split = p.k_blocks;
  int block_q = plan.block_q;
  if (plan.pairs) best_width(M, N, false, &block_q);  // the single-CTA kernel was forced
  if (epilogue == EPI_SWIGLU_BF16) block_q = (block_q + 31) / 32 * 32 > 256 ? 256 : (block_q + 31) / 32 * 32;
  if (!cached_map(&map_row, x, M, K, ldx, BLOCK_P) || !cached_map(&map_col, w, N, K, ldw, block_q))
    return TL_ERR_UNSUPPORTED;
  p.block_q = block_q;
  p.row_tiles = (M + BLOCK_P - 1) / BLOCK_P;
  p.num_tiles = p.row_tiles * ((N + block_q - 1) / block_q);
  const int stage_bytes = ROW_TILE_BYTES + block_q * BLOCK_K * 2;
  p.stages = (SMEM_LIMIT - 1024 - 512) / stage_bytes;
  if (p.stages > 8) p.stages = 8;
  const int smem = p.stages * stage_bytes + 1024 + 512;
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(gemm_tc_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           SMEM_LIMIT);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  const int ctas = p.num_tiles < sm_count() ? p.num_tiles : sm_count();
  tl::launch_kernel(gemm_tc_persistent_kernel, dim3(ctas), THREADS, smem, stream, map_row, map_col, p);
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
