// Paged causal grouped-query attention for PROMPT PORTIONS on the 5th-generation tensor
// cores (tcgen05), bfloat16, head_dim 128.
//
// One CTA takes up to 128 PACKED ROWS of one (request, KV head): the pairs (token of the
// step, query head of the KV head's group), token-major, so every key/value tile that is
// loaded serves all query heads of the group.  It walks over the keys in tiles of 128
// absolute positions:
//
//   loader thread   TMA-loads the tile's pages of K and V (one box of page_size x 64
//                   elements per page and half of the head, 128-byte swizzle) through the
//                   block table into a two-stage ring;
//   MMA thread      S = Q K^T   (tcgen05.mma 128 x 128 x 16, Q and K K-major in shared
//                   memory, S in tensor memory, double-buffered) and, one tile behind,
//                   O += P V    (P K-major from shared memory, V as the MN-major operand);
//   softmax warps   eight warps, two threads per row (each half of a tile's keys): read S
//                   from tensor memory, mask by
//                   position, keep the running max and sum in float32, write P as bfloat16
//                   into shared memory, and rescale O in tensor memory when the row's max
//                   has grown by more than 2^8 since O was last scaled (a smaller growth is
//                   carried in P, whose exponent range has room for it).
//
// At the end the softmax warps divide O by the row sums and store bfloat16 output.
// Numerics are those of attention_mma.cu and of the reference's Triton kernel
// (v10_triton_paged_gqa/kernel/gqa.py:91-111): float32 scores scaled by head_dim^-0.5,
// float32 max/sum/accumulator, P rounded to the value dtype before P V.
//
// Every mbarrier wait is bounded (tcgen05.cuh); a wait that gives up records a code that
// tl_attention_tc_error() returns, and the CTA still runs to its end and frees its TMEM.
#include <math.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int D = 128;          // head_dim
constexpr int ROWS = 128;       // packed rows a CTA (UMMA M)
constexpr int KEYS = 128;       // keys a tile (UMMA N of S, K of P V)
constexpr int THREADS = 320;    // warps 0-7 softmax (two per TMEM lane quarter), 8 MMA, 9 loader
constexpr int SLAB = ROWS * 128;  // bytes of a [128 rows][64 bf16] swizzled slab
constexpr int TILE_BYTES = 2 * SLAB;  // a 128 x 128 bf16 operand tile = two slabs
constexpr float RESCALE_THRESHOLD = 8.f;  // log2 units

__device__ int g_error_word = 0;

#ifdef ATTN_TIMING
__device__ unsigned long long g_timing[32];
#define TIMING_BEGIN() long long t_acc[8] = {0, 0, 0, 0, 0, 0, 0, 0}; long long t_last = clock64();
#define TICK(slot) { const long long t_now = clock64(); t_acc[slot] += t_now - t_last; t_last = t_now; }
#define TIMING_END(base) if (lane == 0) { for (int t_i = 0; t_i < 8; ++t_i) atomicAdd(&g_timing[(base) + t_i], (unsigned long long)t_acc[t_i]); }
#else
#define TIMING_BEGIN()
#define TICK(slot)
#define TIMING_END(base)
#endif

struct Params {
  const __nv_bfloat16* q;
  long long q_stride;
  const int* block_table;
  int table_width;
  const int* req_indptr;
  const int* kv_before;
  const int* tile_req;
  const int* tile_row;
  __nv_bfloat16* out;
  long long out_stride;
  int nh, nkv, page_size, window, rows_per_tile;
  float scale_log2;
};

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr(smem)), "l"(gmem), "r"(bytes) : "memory");
}
// 2^x by the special-function unit (ex2.approx: 2 ulp; the result is rounded to bfloat16 anyway).
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Instruction descriptor for O += P V: A (P) K-major, B (V) MN-major (bit 16).
__device__ __forceinline__ uint32_t idesc_pv() { return idesc_bf16_f32(ROWS, D) | (1u << 16); }

// Shared-memory descriptor of the MN-major operand V: a tile is two slabs (halves of the
// head) of [128 keys][64 elements]; 8 keys form a 1024-byte swizzle atom (stride byte
// offset), the slabs are SLAB bytes apart (leading byte offset).
__device__ __forceinline__ uint64_t smem_desc_v(uint32_t saddr) {
  uint64_t desc = 0;
  desc |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  desc |= (uint64_t)(SLAB >> 4) << 16;
  desc |= (uint64_t)(1024 >> 4) << 32;
  desc |= (uint64_t)1 << 46;
  desc |= (uint64_t)2 << 61;
  return desc;
}

__device__ __forceinline__ void tmem_st_32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// float <-> unsigned code whose unsigned order is the floats' order (0 is below every float)
__device__ __forceinline__ uint32_t ordered_code(float f) {
  const uint32_t b = __float_as_uint(f);
  return (b >> 31) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float ordered_value(uint32_t u) {
  return __uint_as_float((u >> 31) ? (u & 0x7fffffffu) : ~u);
}

__global__ void __launch_bounds__(THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_kv, const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_tile = smem;                       // 32 KB
  uint8_t* p_tiles = smem + TILE_BYTES;         // 2 x 32 KB
  uint8_t* k_tiles = smem + 3 * TILE_BYTES;     // 2 x 32 KB
  uint8_t* v_tiles = smem + 5 * TILE_BYTES;     // 2 x 32 KB
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 7 * TILE_BYTES);
  uint64_t* k_full = bars;        // [2]
  uint64_t* v_full = bars + 2;    // [2]
  uint64_t* k_empty = bars + 4;   // [2]
  uint64_t* v_empty = bars + 6;   // [2]
  uint64_t* s_full = bars + 8;    // [2]
  uint64_t* s_empty = bars + 10;  // [2]  (8 arrivals: one per softmax warp)
  uint64_t* p_full = bars + 12;   // [2]  (8 arrivals)
  uint64_t* p_empty = bars + 14;  // [2]  P V of the tile that used this P buffer is done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  // [3][128 rows] row maxima of three consecutive tiles (order-preserving unsigned codes, joined by
  // atomicMax from the two halves), then [2 halves][128] row sums at the end
  uint32_t* exchange = reinterpret_cast<uint32_t*>(tmem_slot + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int req = p.tile_req[blockIdx.x];
  const int row_start = p.tile_row[blockIdx.x];
  const int kvh = blockIdx.y;
  const int g = p.nh / p.nkv;
  const int tok0 = p.req_indptr[req];
  const int q_len = p.req_indptr[req + 1] - tok0;
  const int before = p.kv_before[req];
  const int row_end = min(q_len * g, row_start + p.rows_per_tile);
  const int* table = p.block_table + (size_t)req * p.table_width;
  const int first_tok = row_start / g, last_tok = (max(row_end, row_start + 1) - 1) / g;
  const int hi_key = before + last_tok;
  const int lo_key = p.window > 0 ? max(0, before + first_tok - p.window + 1) : 0;
  const int tile_begin = lo_key / KEYS, tile_end = hi_key / KEYS + 1;
  const int num_tiles = tile_end - tile_begin;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 8);
      mbar_init(&p_full[i], 8);
      mbar_init(&p_empty[i], 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  for (int i = threadIdx.x; i < 3 * ROWS; i += THREADS) exchange[i] = 0u;
  if (threadIdx.x == 0) {
    prefetch_tensormap(&map_kv);
  }
  if (warp == 8) {
    tmem_alloc<512>(tmem_slot);
    tmem_relinquish();
  }
  tl::pdl_launch_dependents();
  tl::pdl_wait();  // q and this step's keys and values come from the preceding kernels

  // ---- Q rows into shared memory in the K-major swizzled layout (all threads)
  for (int i = threadIdx.x; i < ROWS * (D / 8); i += THREADS) {
    const int r = i / (D / 8), c16 = i % (D / 8);
    const int row = row_start + r;
    const bool valid = r < p.rows_per_tile && row < row_end;
    const __nv_bfloat16* src = p.q;
    if (valid) src = p.q + (size_t)(tok0 + row / g) * p.q_stride + (size_t)(kvh * g + row % g) * D + c16 * 8;
    uint8_t* dst = q_tile + (c16 >> 3) * SLAB + r * 128 + (((c16 & 7) ^ (r & 7)) << 4);
    cp_async_16(dst, src, valid);
  }
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
  fence_proxy_async();  // the tensor core reads what ordinary stores and cp.async wrote
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 256;

  if (warp == 9) {
    // ------------------------------------------------------------------ loader
    // Lane l copies half (l & 1) of page (l >> 1) of every tile: a box of page_size keys x 64
    // elements (page_size >= 8, so a tile has at most 16 pages).
    const int pages_per_tile = KEYS / p.page_size;
    const int my_page = lane >> 1, my_half = lane & 1;
    const bool active = my_page < pages_per_tile;
    TIMING_BEGIN();
    for (int j = 0; j < num_tiles; ++j) {
      const int s = j & 1;
      const uint32_t phase = (j >> 1) & 1;
      const int index = (tile_begin + j) * pages_per_tile + my_page;
      const int page = (active && index < p.table_width) ? table[index] : 0;  // beyond the table: page 0
      const uint32_t offset = s * TILE_BYTES + my_half * SLAB + my_page * p.page_size * 128;
      TICK(0);
      mbar_wait(&k_empty[s], phase ^ 1, abort_flag, &g_error_word, 1);
      TICK(1);
      if (lane == 0) mbar_expect_tx(&k_full[s], TILE_BYTES);
      __syncwarp();
      if (active)
        tma_load_2d(k_tiles + offset, &map_kv, &k_full[s], my_half * 64, ((page * 2 + 0) * p.nkv + kvh) * p.page_size);
      TICK(2);
      mbar_wait(&v_empty[s], phase ^ 1, abort_flag, &g_error_word, 2);
      TICK(3);
      if (lane == 0) mbar_expect_tx(&v_full[s], TILE_BYTES);
      __syncwarp();
      if (active)
        tma_load_2d(v_tiles + offset, &map_kv, &v_full[s], my_half * 64, ((page * 2 + 1) * p.nkv + kvh) * p.page_size);
      TICK(4);
    }
    TIMING_END(0);
  } else if (warp == 8) {
    // --------------------------------------------------------------------- MMA
    if (lane == 0) {
      const uint32_t idesc_s = idesc_bf16_f32(ROWS, KEYS);
      const uint32_t idesc_o = idesc_pv();
      const uint32_t q_addr = smem_addr(q_tile);
      TIMING_BEGIN();
      auto issue_pv = [&](int j) {  // O (+)= P_j V_j
        const int s = j & 1;
        TICK(3);
        mbar_wait(&p_full[s], (j >> 1) & 1, abort_flag, &g_error_word, 5);
        TICK(4);
        mbar_wait(&v_full[s], (j >> 1) & 1, abort_flag, &g_error_word, 6);
        TICK(5);
        fence_after_sync();
        const uint32_t v_addr = smem_addr(v_tiles + s * TILE_BYTES);
        const uint32_t p_addr = smem_addr(p_tiles + s * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < KEYS / 16; ++k) {
          const uint64_t a_desc = smem_desc_sw128(p_addr + (k >> 2) * SLAB + (k & 3) * 32);
          const uint64_t b_desc = smem_desc_v(v_addr + k * 2048);  // 16 keys = two 8-key atoms
          mma_bf16(tmem_o, a_desc, b_desc, idesc_o, j > 0 || k > 0);
        }
        mma_commit(&v_empty[s]);
        mma_commit(&p_empty[s]);
        TICK(6);
      };
      for (int j = 0; j < num_tiles; ++j) {
        const int s = j & 1;
        const uint32_t phase = (j >> 1) & 1;
        TICK(0);
        mbar_wait(&k_full[s], phase, abort_flag, &g_error_word, 3);
        TICK(1);
        mbar_wait(&s_empty[s], phase ^ 1, abort_flag, &g_error_word, 4);
        TICK(2);
        fence_after_sync();
        const uint32_t k_addr = smem_addr(k_tiles + s * TILE_BYTES);
#pragma unroll
        for (int k = 0; k < D / 16; ++k) {
          const uint64_t a_desc = smem_desc_sw128(q_addr + (k >> 2) * SLAB + (k & 3) * 32);
          const uint64_t b_desc = smem_desc_sw128(k_addr + (k >> 2) * SLAB + (k & 3) * 32);
          mma_bf16(tmem_base + s * KEYS, a_desc, b_desc, idesc_s, k > 0);
        }
        mma_commit(&k_empty[s]);
        mma_commit(&s_full[s]);
        if (j > 0) issue_pv(j - 1);  // one tile behind, so S of this tile overlaps the softmax of the last
      }
      if (num_tiles > 0) issue_pv(num_tiles - 1);
      TIMING_END(8);
    }
  } else {
    // ----------------------------------------------------------------- softmax
    // Two threads a row: warps 0-3 take keys (and output columns) 0-63 of every tile, warps
    // 4-7 take 64-127; the halves agree on the row's maximum through shared memory.
    const int quarter = warp & 3, half = warp >> 2;
    const int r = quarter * 32 + lane;  // row of the tile = lane of tensor memory
    const int row = row_start + r;
    const bool row_valid = r < p.rows_per_tile && row < row_end;
    const int pos = row_valid ? before + row / g : -1;
    const int lo = (row_valid && p.window > 0) ? max(0, pos - p.window + 1) : 0;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    constexpr int HALF = KEYS / 2;
    float m_ref = -INFINITY, l_sum = 0.f;  // m_ref in log2 units (already scaled); l_sum of this half
    TIMING_BEGIN();
    for (int j = 0; j < num_tiles; ++j) {
      const int s = j & 1;
      TICK(0);
      const int key0 = (tile_begin + j) * KEYS + half * HALF;  // first key of this thread's half
      mbar_wait(&s_full[s], (j >> 1) & 1, abort_flag, &g_error_word, 7);
      TICK(1);
      fence_after_sync();
      const uint32_t s_addr = tmem_base + s * KEYS + half * HALF + lane_base;
      // A half tile whose keys are all visible to every row of this warp needs no masking
      const bool visible = key0 + HALF - 1 <= pos && key0 >= lo;
      const bool warp_visible = __all_sync(0xffffffffu, visible);
      // pass 1: the row's maximum over the keys of this half (in raw score units)
      float m_a = -INFINITY, m_b = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < HALF; c += 32) {
        uint32_t v[32];
        tmem_ld_32(s_addr + c, v);
        tmem_ld_wait();
        if (warp_visible) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            m_a = fmaxf(m_a, __uint_as_float(v[i]));
            m_b = fmaxf(m_b, __uint_as_float(v[i + 1]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = key0 + c + i;
            if (key <= pos && key >= lo) m_a = fmaxf(m_a, __uint_as_float(v[i]));
          }
        }
      }
      TICK(2);
      // Both halves join their maxima in the tile's slot; the slot of the tile after next was last
      // read before the previous barrier and is written again only after the next one.
      atomicMax(&exchange[(j % 3) * ROWS + r], ordered_code(fmaxf(m_a, m_b)));
      asm volatile("bar.sync 1, 256;" ::: "memory");  // the eight softmax warps
      const float m_tile = ordered_value(exchange[(j % 3) * ROWS + r]) * p.scale_log2;  // the scale is positive
      if (half == 0) exchange[((j + 2) % 3) * ROWS + r] = 0u;
      // the reference max moves only when the row's max has grown past the threshold
      float factor = 1.f;
      bool rescale = false;
      if (m_tile > m_ref + RESCALE_THRESHOLD || (m_ref == -INFINITY && m_tile > -INFINITY)) {
        factor = m_ref == -INFINITY ? 0.f : exp2f(m_ref - m_tile);
        rescale = m_ref != -INFINITY;
        m_ref = m_tile;
      }
      l_sum *= factor;
      TICK(3);
      // this tile's P buffer is free once P V of the tile before last is done
      mbar_wait(&p_empty[s], ((j >> 1) & 1) ^ 1, abort_flag, &g_error_word, 8);
      TICK(4);
      if (__any_sync(0xffffffffu, rescale)) {
        // O may only be touched when no P V is in flight: wait for the previous tile's
        mbar_wait(&p_empty[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, &g_error_word, 10);
        fence_after_sync();
#pragma unroll 1
        for (int c = 0; c < D / 2; c += 32) {  // this thread's half of the output columns
          uint32_t v[32];
          tmem_ld_32(tmem_o + lane_base + half * (D / 2) + c, v);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * factor);
          tmem_st_32(tmem_o + lane_base + half * (D / 2) + c, v);
        }
        tmem_st_wait();
      }
      TICK(5);
      // pass 2: P = exp2(S * scale - m_ref), row sum, P as bfloat16 into shared memory
      const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
      float sum_a = 0.f, sum_b = 0.f;
#pragma unroll 1
      for (int c = 0; c < HALF; c += 32) {
        uint32_t v[32];
        tmem_ld_32(s_addr + c, v);
        tmem_ld_wait();
        uint32_t packed[16];
        if (warp_visible) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float a = fast_exp2(fmaf(__uint_as_float(v[i]), p.scale_log2, neg_m));
            const float b = fast_exp2(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, neg_m));
            sum_a += a;
            sum_b += b;
            __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
            packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const int key = key0 + c + i;
            const float a = (key <= pos && key >= lo) ? fast_exp2(fmaf(__uint_as_float(v[i]), p.scale_log2, neg_m)) : 0.f;
            const float b = (key + 1 <= pos && key + 1 >= lo)
                                ? fast_exp2(fmaf(__uint_as_float(v[i + 1]), p.scale_log2, neg_m)) : 0.f;
            sum_a += a;
            sum_b += b;
            __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
            packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
          }
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4) {  // four 16-byte chunks of 8 keys; a half is one slab
          const int c8 = (c >> 3) + q4;
          uint8_t* dst = p_tiles + s * TILE_BYTES + half * SLAB + r * 128 + (((c8 & 7) ^ (r & 7)) << 4);
          *reinterpret_cast<uint4*>(dst) = make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
        }
      }
      l_sum += sum_a + sum_b;
      TICK(6);
      fence_proxy_async();   // P is read by the tensor core
      fence_before_sync();   // our tcgen05.ld/st of S and O are done
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[s]);
        mbar_arrive(&p_full[s]);
      }
      TICK(7);
    }
    if (warp == 0) TIMING_END(16);
    if (warp == 4) TIMING_END(24);
    // ---- output: O / l (the two halves add their sums)
    float* sums = reinterpret_cast<float*>(exchange);
    asm volatile("bar.sync 1, 256;" ::: "memory");  // the last tile's maxima have been read
    sums[half * ROWS + r] = l_sum;
    asm volatile("bar.sync 1, 256;" ::: "memory");
    const float l_all = sums[r] + sums[ROWS + r];
    if (num_tiles > 0)
      mbar_wait(&p_empty[(num_tiles - 1) & 1], ((num_tiles - 1) >> 1) & 1, abort_flag, &g_error_word, 9);
    fence_after_sync();
    const float inv = l_all > 0.f ? 1.f / l_all : 0.f;
    __nv_bfloat16* dst = nullptr;
    if (row_valid)
      dst = p.out + (size_t)(tok0 + row / g) * p.out_stride + (size_t)(kvh * g + row % g) * D + half * (D / 2);
#pragma unroll 1
    for (int c = 0; c < D / 2; c += 32) {
      uint32_t v[32];
      tmem_ld_32(tmem_o + lane_base + half * (D / 2) + c, v);
      tmem_ld_wait();
      if (row_valid && num_tiles > 0) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[i]) * inv, __uint_as_float(v[i + 1]) * inv);
          packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
        }
#pragma unroll
        for (int q4 = 0; q4 < 4; ++q4)
          *reinterpret_cast<uint4*>(dst + c + 8 * q4) =
              make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
      }
    }
  }
  __syncwarp();
  fence_before_sync();
  __syncthreads();
  if (warp == 8) {
    fence_after_sync();
    tmem_dealloc<512>(tmem_base);
  }
}

// ------------------------------------------------------------------ host side
struct MapKey {
  const void* base;
  uint64_t rows;
  uint32_t box_rows;
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && box_rows == o.box_rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return (reinterpret_cast<size_t>(k.base) * 1000003u ^ k.rows) * 1000003u ^ k.box_rows;
  }
};

bool cached_map(CUtensorMap* out, const void* base, uint64_t rows, uint32_t box_rows) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex lock;
  const MapKey key{base, rows, box_rows};
  std::lock_guard<std::mutex> guard(lock);
  auto it = cache.find(key);
  if (it == cache.end()) {
    CUtensorMap map;
    if (!tc_host::make_map_bf16(&map, base, rows, D, D, box_rows)) return false;
    if (cache.size() > 1024) cache.clear();
    it = cache.emplace(key, map).first;
  }
  *out = it->second;
  return true;
}

}  // namespace

extern "C" {

#ifdef ATTN_TIMING
int tl_attention_tc_timing(unsigned long long* out) {  // reads and clears the 32 counters
  unsigned long long zero[32] = {};
  if (cudaMemcpyFromSymbol(out, g_timing, sizeof(zero)) != cudaSuccess) return -1;
  return (int)cudaMemcpyToSymbol(g_timing, zero, sizeof(zero));
}
#endif

int tl_attention_tc_error() {
  int value = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&value, g_error_word, sizeof(int)) != cudaSuccess) return -1;
  if (value) cudaMemcpyToSymbol(g_error_word, &zero, sizeof(int));
  return value;
}

// Packed rows a tile holds for a group of ``group`` query heads (whole tokens only).
int tl_attention_tc_rows(int group) { return group > 0 && group <= ROWS ? (ROWS / group) * group : 0; }

// pages: one cache layer [num_pages][2][nkv][page_size][128] bf16.  tile_req / tile_row:
// request and first packed row (a multiple of tl_attention_tc_rows(nh / nkv)) of each tile.
int tl_attention_tc(const void* q, long long q_stride, const void* pages, long long num_pages,
                    const int* block_table, int table_width, const int* req_indptr, const int* kv_before,
                    const int* tile_req, const int* tile_row, int tiles, void* out, long long out_stride, int nh,
                    int nkv, int d, int page_size, int window, float scale, cudaStream_t stream) {
  if (tiles <= 0) return 0;
  if (d != D || nkv <= 0 || nh % nkv || nh / nkv > ROWS || page_size < 8 || page_size > KEYS || KEYS % page_size ||
      q_stride % 8 || out_stride % 8 || nkv > 65535 || !tile_req || !tile_row)
    return TL_ERR_UNSUPPORTED;
  CUtensorMap map_kv;
  if (!cached_map(&map_kv, pages, (uint64_t)num_pages * 2 * nkv * page_size, (uint32_t)page_size))
    return TL_ERR_UNSUPPORTED;
  Params p;
  p.q = (const __nv_bfloat16*)q;
  p.q_stride = q_stride;
  p.block_table = block_table;
  p.table_width = table_width;
  p.req_indptr = req_indptr;
  p.kv_before = kv_before;
  p.tile_req = tile_req;
  p.tile_row = tile_row;
  p.out = (__nv_bfloat16*)out;
  p.out_stride = out_stride;
  p.nh = nh;
  p.nkv = nkv;
  p.page_size = page_size;
  p.window = window;
  p.rows_per_tile = tl_attention_tc_rows(nh / nkv);
  p.scale_log2 = scale * 1.4426950408889634f;
  constexpr int SMEM = 7 * TILE_BYTES + 1024 + 256 + 3 * ROWS * 4;
  static_assert(SMEM <= 232448, "shared memory of one CTA");
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attention_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  tl::launch_kernel(attention_tc_kernel, dim3(tiles, nkv), THREADS, SMEM, stream, map_kv, p);
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
