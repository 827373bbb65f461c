// Paged causal grouped-query attention on tensor cores for bfloat16, head_dim 64 or 128.
//
// Work is cut into tiles of PACKED ROWS: for one (request, KV head) the rows are the
// pairs (token of the step, query head of the KV head's group), token-major, so that all
// query heads of a group share every K/V tile that is loaded.  A CTA of 4 warps walks
// over the keys in tiles of 64 absolute positions (pages gathered through the block
// table with cp.async into swizzled shared memory, double-buffered), computes
// S = Q K^T with mma.sync.m16n8k16 (bf16 in, float32 out), keeps the online-softmax
// state (max, sum, accumulator) in float32 registers, and accumulates P V with P
// rounded to bfloat16 as the tensor-core operand.
//
// Two shapes of CTA:
//   ROWS64  (prompt portions): the tile has 64 packed rows, each warp owns 16 of them
//           and sees every key of the tile.
//   ROWS16  (decode, few rows a request): the tile has 16 packed rows that all four
//           warps share; each warp takes 16 of the tile's 64 keys, and the warps' partial
//           states are merged at the end.  The keys of a request can also be split over
//           blockIdx.z; each split then writes its (max, sum, accumulator) to a workspace
//           and a second kernel merges the splits.
//
// Decode tiles (ROWS16) with a page size that is a multiple of 8 and divides 64 get their keys
// and values by TMA instead: one box of page_size x 64 elements per page, K or V and half of the
// head, one lane of warp 0 a box, into the 128-byte-swizzled layout that ldmatrix reads without
// bank conflicts; the warps wait on an mbarrier per stage (bounded; a wait that gives up leaves a
// code that tl_attention_mma_error() returns).  The gather with cp.async costs every thread some
// hundred instructions a tile, which is what the 16-row tiles spent most of their time on.
//
// Reference counterparts: forward_ragged_attention_kernel and
// forward_slot_attention_decode_kernel (v10_triton_paged_gqa/kernel/gqa.py:5-228), which
// use the same numerics: float32 scores scaled by head_dim^-0.5, float32 max/sum/acc, the
// weights cast to the value dtype before P.V, acc / sum at the end.
#include <math.h>

#include <mutex>
#include <type_traits>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

__device__ int g_error_word = 0;

constexpr int WARPS = 4;
constexpr int THREADS = WARPS * 32;
constexpr int BLOCK_N = 64;  // keys per tile

struct Params {
  const __nv_bfloat16* q;  // packed qkv rows; query head h of token t at q + t*q_stride + h*D
  long long q_stride;
  const __nv_bfloat16* pages;  // [page][2][nkv][page_size][D]
  const int* block_table;      // [requests][table_width]
  int table_width;
  const int* req_indptr;  // [requests + 1] first token of each request in the step
  const int* kv_before;   // [requests] cached tokens before the step
  const int* tile_req;    // [tiles] request of each row tile, or null: tile i = request i
  const int* tile_row;    // [tiles] first packed row of the tile (null: 0)
  __nv_bfloat16* out;     // [tokens][nh*D]
  long long out_stride;
  float* part_acc;  // [tiles*nh][splits][D]   (splits > 1: decode tiles of one token each)
  float* part_ml;   // [tiles*nh][splits][2]
  int* arrivals;    // [tiles*nkv] zero between launches: splits of a (tile, KV head) that have written (null: a second kernel merges)
  int nh, nkv, page_size, window, splits;
  int num_pages;   // pages in the pool (checked in the debug build)
  int page_shift;  // log2(page_size) when it is a power of two, else -1
  int overlap_max_tiles;  // host only: overlapped launch up to this many row tiles
  int late_wait;  // the kernel before this one has itself waited for q, keys and values: start at once, wait for it at the end
  float scale_log2;  // scale * log2(e)
};

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  const int bytes = valid ? 16 : 0;  // 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(s));
}
__device__ __forceinline__ void mma_16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&h);
}

// Element (row, 8-element chunk) of a [rows][D] bf16 tile with the chunk index xor-ed by
// the row, so that the 8 rows of an ldmatrix fall into different banks.
template <int D> __device__ __forceinline__ __nv_bfloat16* tile_at(__nv_bfloat16* tile, int row, int chunk) {
  return tile + row * D + ((chunk ^ (row & 7)) << 3);
}

// The same for a [64][D] key or value tile: with TMA the tile is D / 64 slabs of [64 rows][64
// elements], each row 128 bytes with its 16-byte chunks xor-ed by the row (the 128-byte swizzle
// of the copy); for D = 64 the two layouts are one.
template <int D, bool TMA> __device__ __forceinline__ __nv_bfloat16* kv_at(__nv_bfloat16* tile, int row, int chunk) {
  if constexpr (TMA) return tile + (chunk >> 3) * (BLOCK_N * 64) + row * 64 + (((chunk & 7) ^ (row & 7)) << 3);
  return tile_at<D>(tile, row, chunk);
}

// Requests the K and V pages of keys [tile * 64, tile * 64 + 64) of one KV head by TMA into a
// stage (warp 0, one lane a box).  Pages past the request's last key or past the table are
// read from page 0 (always there; their keys are masked and their value rows are cleared in
// shared memory before use).
template <int D>
__device__ __forceinline__ void tma_kv_tile(const CUtensorMap* map, const Params& p, const int* table, int kvh, int tile,
                                            int hi_key, __nv_bfloat16* stage, uint64_t* full, int lane) {
  constexpr int SLABS = D / 64;
  const int pages_per_tile = BLOCK_N / p.page_size;
  const int boxes = pages_per_tile * 2 * SLABS;  // at most 8 * 2 * 2 = 32
  if (lane == 0) tc::mbar_expect_tx(full, 2 * BLOCK_N * D * 2);
  __syncwarp();
  if (lane < boxes) {
    const int slab = lane % SLABS, is_v = (lane / SLABS) & 1, page_i = lane / (2 * SLABS);
    const int index = tile * pages_per_tile + page_i;
    const bool wanted = index < p.table_width && index * p.page_size <= hi_key;
    const int page = wanted ? table[index] : 0;
    __nv_bfloat16* dst = stage + is_v * (BLOCK_N * D) + slab * (BLOCK_N * 64) + page_i * p.page_size * 64;
    tc::tma_load_2d(dst, map, full, slab * 64, ((page * 2 + is_v) * p.nkv + kvh) * p.page_size);
  }
}

// Gathers the K and V rows of keys [key0, key0 + 64) of one KV head into shared memory.
// Rows outside [lo_key, hi_key] are zero-filled instead of read.
template <int D>
__device__ __forceinline__ void load_kv_tile(const Params& p, const int* table, int kvh, int key0, int lo_key,
                                             int hi_key, __nv_bfloat16* ks, __nv_bfloat16* vs) {
  constexpr int CHUNKS = D / 8;                   // 16-byte chunks in a row
  constexpr int ROWS_PER_PASS = THREADS / CHUNKS;  // each thread keeps its chunk column
  constexpr int PASSES = BLOCK_N / ROWS_PER_PASS;
  const size_t page_elems = (size_t)2 * p.nkv * p.page_size * D;
  const size_t v_off = (size_t)p.nkv * p.page_size * D;
  const int c = threadIdx.x % CHUNKS, r0 = threadIdx.x / CHUNKS;
  // first the page of every row (independent loads), then the copies
  int page[PASSES], slot[PASSES];
#pragma unroll
  for (int k = 0; k < PASSES; ++k) {
    const int key = key0 + r0 + k * ROWS_PER_PASS;
    const bool valid = key >= lo_key && key <= hi_key;
    int index, within;
    if (p.page_shift >= 0) {
      index = key >> p.page_shift;
      within = key & (p.page_size - 1);
    } else {
      index = key / p.page_size;
      within = key - index * p.page_size;
    }
    // debug build: a key beyond the table or a page outside the pool is skipped (zero-filled) and recorded
    const bool in_table = TL_DEBUG_OK(!valid || index < p.table_width, TL_DEBUG_POSITION, key);
    page[k] = (valid && in_table) ? table[index] : -1;
    if (page[k] >= 0 && !TL_DEBUG_OK(page[k] < p.num_pages, TL_DEBUG_PAGE, page[k])) page[k] = -1;
    slot[k] = within;
  }
#pragma unroll
  for (int k = 0; k < PASSES; ++k) {
    const int r = r0 + k * ROWS_PER_PASS;
    const bool valid = page[k] >= 0;
    const __nv_bfloat16* src = p.pages;
    if (valid) src = p.pages + (size_t)page[k] * page_elems + ((size_t)kvh * p.page_size + slot[k]) * D + c * 8;
    cp_async_16(tile_at<D>(ks, r, c), src, valid);
    cp_async_16(tile_at<D>(vs, r, c), valid ? src + v_off : src, valid);
  }
}

// Key splits a request really uses out of the ``splits`` CTAs the grid holds for it: no split
// shorter than three key tiles (192 keys).  The grid is sized on the host for the longest request it
// may meet (under a CUDA graph: the longest the engine allows); a request's own count follows from
// its length on the device, and the CTAs beyond it leave at once.
constexpr int MIN_TILES_A_SPLIT = 3;  // 192 keys (measured against 128 and 256: -0.4 to -0.9 % of a decode step at batch 1 to 4)
__device__ __forceinline__ int effective_splits(int splits, int key_tiles) {
  return min(splits, max(1, (key_tiles + MIN_TILES_A_SPLIT - 1) / MIN_TILES_A_SPLIT));
}

// STAGES: key/value tiles in shared memory; 2, or 3 with the TMA loader where the grid leaves
// room for only two CTAs an SM anyway.
template <int D, bool ROWS16, bool TMA, int STAGES>
__global__ void __launch_bounds__(THREADS, STAGES == 2 ? 3 : 2)
attention_mma_kernel(const __grid_constant__ CUtensorMap map_kv, const Params p) {
  static_assert(!TMA || ROWS16, "the TMA loader serves the 16-row tiles");
  static_assert(STAGES == 2 || TMA, "more than two stages need the TMA loader");
  // The wait on the preceding kernel comes further down: the step's metadata is written
  // by a host copy before any kernel of the step, and key/value tiles that lie wholly
  // before the step's own tokens were written by earlier steps, so both may be read first.
  constexpr int BLOCK_M = ROWS16 ? 16 : 64;
  constexpr int KSTEPS = D / 16;   // k-steps of Q K^T
  constexpr int DTILES = D / 8;    // n-tiles of the output
  // key sub-range of a 64-key tile this warp multiplies: all of it, or its own 16 keys
  constexpr int WARP_KEYS = ROWS16 ? 16 : 64;
  constexpr int NTILES = WARP_KEYS / 8;

  // Shared memory: 2 stages x (K, V) x [64][D].  The Q rows are first loaded into the
  // second stage's space; once every warp holds its Q fragments in registers that space
  // is free for the key/value tiles, so three CTAs fit an SM.
  extern __shared__ __align__(128) uint8_t smem_raw[];
  // the swizzle of the TMA copies works on address bits: the stages start on a 1024-byte boundary
  uint8_t* smem_base = TMA ? reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023)
                           : smem_raw;
  __nv_bfloat16* kv = reinterpret_cast<__nv_bfloat16*>(smem_base);
  // 64-row tiles: Q [64][D] inside stage 1.  16-row tiles (decode): Q [16][D] after the
  // stages, so that both stages can be filled before the wait on the preceding kernel.
  __nv_bfloat16* qs = ROWS16 ? kv + STAGES * 2 * BLOCK_N * D : kv + 2 * BLOCK_N * D;
  // TMA: one "tile has landed" barrier a stage and the block's "a wait gave up" word, after Q
  uint64_t* full = reinterpret_cast<uint64_t*>(qs + BLOCK_M * D);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(full + STAGES);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int req = p.tile_req ? p.tile_req[blockIdx.x] : blockIdx.x;
  const int row_start = p.tile_row ? p.tile_row[blockIdx.x] : 0;
  const int kvh = blockIdx.y;
  const int split = blockIdx.z;
  const int g = p.nh / p.nkv;
  const int tok0 = p.req_indptr[req];
  const int q_len = p.req_indptr[req + 1] - tok0;
  const int before = p.kv_before[req];
  const int total_rows = q_len * g;
  const int* table = p.block_table + (size_t)req * p.table_width;

  // rows of this tile: [row_start, row_end)
  const int row_end = min(total_rows, row_start + BLOCK_M);
  if (row_start >= row_end) {
    tl::pdl_wait();
    return;
  }
  const int first_tok = row_start / g, last_tok = (row_end - 1) / g;
  const int hi_key = before + last_tok;  // last key any row of the tile may see
  int lo_key = 0;
  if (p.window > 0) lo_key = max(0, before + first_tok - p.window + 1);

  // key tiles of this CTA
  int tile_begin = lo_key / BLOCK_N, tile_end = hi_key / BLOCK_N + 1;
  int my_splits = 1;
  if (p.splits > 1) {
    my_splits = effective_splits(p.splits, tile_end - tile_begin);
    if (split >= my_splits) {  // the request is too short to need this CTA
      tl::pdl_wait();
      return;
    }
    const int per = (tile_end - tile_begin + my_splits - 1) / my_splits;
    tile_begin = tile_begin + split * per;
    tile_end = min(tile_end, tile_begin + per);
  }
  if constexpr (TMA) {
    if (threadIdx.x == 0) {
      for (int i = 0; i < STAGES; ++i) tc::mbar_init(&full[i], 1);
      *abort_flag = 0;
      tc::mbar_fence_init();
      tc::prefetch_tensormap(&map_kv);
    }
    __syncthreads();
  }

  // ---- key/value tiles that earlier steps wrote may be requested before the wait
  constexpr int STAGE_ELEMS = 2 * BLOCK_N * D;
  const int num_tiles = max(0, tile_end - tile_begin);
  int issued = 0;  // tiles requested so far, counted from tile_begin
  if constexpr (ROWS16) {
    while (issued < min(STAGES, num_tiles) && (tile_begin + issued) * BLOCK_N + BLOCK_N - 1 < before) {
      __nv_bfloat16* stage = kv + issued * STAGE_ELEMS;
      if constexpr (TMA) {
        if (warp == 0) tma_kv_tile<D>(&map_kv, p, table, kvh, tile_begin + issued, hi_key, stage, &full[issued], lane);
      } else {
        load_kv_tile<D>(p, table, kvh, (tile_begin + issued) * BLOCK_N, lo_key, hi_key, stage, stage + BLOCK_N * D);
        cp_async_commit();
      }
      ++issued;
    }
  }
  // q and this step's keys and values are written and visible after the wait.  With late_wait the
  // kernel before this one is the prompt portions' attention, which is independent of this one and
  // whose every CTA had waited for them before this grid could start: the wait moves to the end.
  if (!p.late_wait) tl::pdl_wait();
  tl::pdl_launch_dependents();  // the next kernel may start its own prologue

  // ---- Q rows into shared memory (zero for rows past the tile's end)
  for (int i = threadIdx.x; i < BLOCK_M * (D / 8); i += THREADS) {
    const int r = i / (D / 8), c = i % (D / 8);
    const int row = row_start + r;
    const bool valid = row < row_end;
    const __nv_bfloat16* src = p.q;
    if (valid) src = p.q + (size_t)(tok0 + row / g) * p.q_stride + (size_t)(kvh * g + row % g) * D + c * 8;
    cp_async_16(tile_at<D>(qs, r, c), src, valid);
  }
  cp_async_commit();
  if (issued == 0 && num_tiles > 0) {
    if constexpr (TMA) {
      if (warp == 0) tma_kv_tile<D>(&map_kv, p, table, kvh, tile_begin, hi_key, kv, &full[0], lane);
    } else {
      load_kv_tile<D>(p, table, kvh, tile_begin * BLOCK_N, lo_key, hi_key, kv, kv + BLOCK_N * D);
    }
    issued = 1;
  }
  cp_async_commit();

  const int my_rows = ROWS16 ? 0 : warp * 16;  // first tile row of this warp
  // the two rows this thread holds in accumulator fragments
  int row_pos[2], row_lo[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const int row = row_start + my_rows + (lane >> 2) + 8 * h;
    if (row < row_end) {
      row_pos[h] = before + row / g;
      row_lo[h] = p.window > 0 ? max(0, row_pos[h] - p.window + 1) : 0;
    } else {
      row_pos[h] = -1;  // sees no key
      row_lo[h] = 0;
    }
  }

  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o_acc[DTILES][4];
#pragma unroll
  for (int i = 0; i < DTILES; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;

  cp_async_wait<0>();  // Q (and what was requested so far) has landed
  __syncthreads();

  unsigned q_frag[KSTEPS][4];
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    const int r = my_rows + (lane & 7) + ((lane >> 3) & 1) * 8;
    const int c = 2 * ks + (lane >> 4);
    ldmatrix_x4(q_frag[ks], tile_at<D>(qs, r, c));
  }
  __syncthreads();  // stage 1 may now be overwritten by key/value tiles

  // the only tiles that can hold rows of keys outside [lo_key, hi_key]
  const int edge_hi_tile = hi_key / BLOCK_N, edge_lo_tile = lo_key > 0 ? lo_key / BLOCK_N : -1;
  // One key tile.  EDGE: the tile may hold rows of keys outside [lo_key, hi_key] (only the first
  // and the last tile of a request can); the common tiles run a body without that code.
  auto process_tile = [&](const int tile, auto edge_tag) {
    constexpr bool EDGE = decltype(edge_tag)::value;
    const int index = tile - tile_begin;
    const int stage = index % STAGES;
    __nv_bfloat16* ks_tile = kv + stage * STAGE_ELEMS;
    __nv_bfloat16* vs_tile = ks_tile + BLOCK_N * D;
    if constexpr (TMA) {
      // keep STAGES tiles requested: the stage of tile index - 1 is free since the barrier that ended it
      while (issued < min(num_tiles, index + STAGES)) {
        const int s_next = issued % STAGES;
        if (warp == 0)
          tma_kv_tile<D>(&map_kv, p, table, kvh, tile_begin + issued, hi_key, kv + s_next * STAGE_ELEMS, &full[s_next], lane);
        ++issued;
      }
    } else if (issued == index + 1 && index + 1 < num_tiles) {  // request the next tile into the other stage
      __nv_bfloat16* next = kv + (stage ^ 1) * STAGE_ELEMS;
      load_kv_tile<D>(p, table, kvh, (tile + 1) * BLOCK_N, lo_key, hi_key, next, next + BLOCK_N * D);
      ++issued;
    }
    if constexpr (TMA) {
      tc::mbar_wait(&full[stage], (index / STAGES) & 1, abort_flag, &g_error_word, 1);  // this tile is here
      // Whole pages were copied: value rows of keys outside [lo_key, hi_key] hold whatever the page
      // held before (another request's values, page 0).  Their weights are exactly 0, but 0 x NaN
      // is NaN, so the warp clears those of its own 16 rows before it multiplies.
      if constexpr (EDGE) {
        const int key_first = tile * BLOCK_N + warp * 16;
        if (key_first + 15 > hi_key || key_first < lo_key) {
          for (int i = lane; i < 16 * (D / 8); i += 32) {
            const int r = i / (D / 8), c = i % (D / 8);
            if (key_first + r > hi_key || key_first + r < lo_key)
              *reinterpret_cast<uint4*>(kv_at<D, true>(vs_tile, warp * 16 + r, c)) = make_uint4(0u, 0u, 0u, 0u);
          }
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // a later TMA copy may refill the stage
          __syncwarp();
        }
      }
    } else {
      cp_async_commit();
      cp_async_wait<1>();  // everything but the request just made has landed: this tile is here
      __syncthreads();
    }

    const int key_base = tile * BLOCK_N + (ROWS16 ? warp * 16 : 0);  // first key this warp multiplies
    const int key_row0 = ROWS16 ? warp * 16 : 0;                      // its row inside the tile

    // ---- S = Q K^T over this warp's keys
    float s[NTILES][4];
#pragma unroll
    for (int i = 0; i < NTILES; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
      for (int nb = 0; nb < NTILES / 2; ++nb) {
        unsigned b[4];
        const int r = key_row0 + nb * 16 + (lane & 7) + (lane >> 4) * 8;
        const int c = 2 * ks + ((lane >> 3) & 1);
        ldmatrix_x4(b, kv_at<D, TMA>(ks_tile, r, c));
        mma_16816(s[2 * nb], q_frag[ks], b[0], b[1]);
        mma_16816(s[2 * nb + 1], q_frag[ks], b[2], b[3]);
      }
    }

    // ---- mask, online softmax (float32)
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int i = 0; i < NTILES; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int h = e >> 1;
        const int key = key_base + i * 8 + (lane & 3) * 2 + (e & 1);
        const bool ok = key <= row_pos[h] && key >= row_lo[h];
        s[i][e] = ok ? s[i][e] * p.scale_log2 : -INFINITY;
        tile_max[h] = fmaxf(tile_max[h], s[i][e]);
      }
    }
    float corr[2], m_use[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 1));
      tile_max[h] = fmaxf(tile_max[h], __shfl_xor_sync(0xffffffffu, tile_max[h], 2));
      const float m_new = fmaxf(m_run[h], tile_max[h]);
      m_use[h] = m_new == -INFINITY ? 0.f : m_new;  // a row that has seen no key yet
      corr[h] = exp2f(m_run[h] - m_use[h]);         // exp2(-inf) = 0 on the first tile
      m_run[h] = m_new;
    }
    float row_sum[2] = {0.f, 0.f};
    unsigned p_frag[NTILES / 2][4];
#pragma unroll
    for (int i = 0; i < NTILES; ++i) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float pv = exp2f(s[i][e] - m_use[e >> 1]);
        s[i][e] = pv;
        row_sum[e >> 1] += pv;
      }
    }
#pragma unroll
    for (int j = 0; j < NTILES / 2; ++j) {
      p_frag[j][0] = pack_bf16(s[2 * j][0], s[2 * j][1]);
      p_frag[j][1] = pack_bf16(s[2 * j][2], s[2 * j][3]);
      p_frag[j][2] = pack_bf16(s[2 * j + 1][0], s[2 * j + 1][1]);
      p_frag[j][3] = pack_bf16(s[2 * j + 1][2], s[2 * j + 1][3]);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 1);
      row_sum[h] += __shfl_xor_sync(0xffffffffu, row_sum[h], 2);
      l_run[h] = l_run[h] * corr[h] + row_sum[h];
    }
#pragma unroll
    for (int i = 0; i < DTILES; ++i) {
      o_acc[i][0] *= corr[0];
      o_acc[i][1] *= corr[0];
      o_acc[i][2] *= corr[1];
      o_acc[i][3] *= corr[1];
    }

    // ---- O += P V over this warp's keys
#pragma unroll
    for (int kk = 0; kk < NTILES / 2; ++kk) {
#pragma unroll
      for (int nb = 0; nb < DTILES / 2; ++nb) {
        unsigned b[4];
        const int r = key_row0 + kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int c = 2 * nb + (lane >> 4);
        ldmatrix_x4_trans(b, kv_at<D, TMA>(vs_tile, r, c));
        mma_16816(o_acc[2 * nb], p_frag[kk], b[0], b[1]);
        mma_16816(o_acc[2 * nb + 1], p_frag[kk], b[2], b[3]);
      }
    }
    __syncthreads();  // the stage may be overwritten by the load after next
  };
  for (int tile = tile_begin; tile < tile_end; ++tile) {
    if (TMA && (tile == edge_hi_tile || tile == edge_lo_tile))
      process_tile(tile, std::true_type{});
    else
      process_tile(tile, std::false_type{});
  }
  cp_async_wait<0>();

  // ---- finish: merge the warps (ROWS16), then write output or split partials
  float* merge = reinterpret_cast<float*>(kv);  // reuse the K/V stages
  if constexpr (ROWS16) {
    __syncthreads();
    // merge[w][row][D + 2]: acc, then max and sum
    constexpr int STRIDE = D + 2;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int r = (lane >> 2) + 8 * h;
      float* dst = merge + ((size_t)warp * 16 + r) * STRIDE;
#pragma unroll
      for (int i = 0; i < DTILES; ++i) {
        dst[i * 8 + (lane & 3) * 2] = o_acc[i][2 * h];
        dst[i * 8 + (lane & 3) * 2 + 1] = o_acc[i][2 * h + 1];
      }
      if ((lane & 3) == 0) {
        dst[D] = m_run[h];
        dst[D + 1] = l_run[h];
      }
    }
    __syncthreads();
    const int rows_here = row_end - row_start;
    for (int i = threadIdx.x; i < rows_here * D; i += THREADS) {
      const int r = i / D, c = i % D;
      float m_all = -INFINITY;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) m_all = fmaxf(m_all, merge[((size_t)w * 16 + r) * STRIDE + D]);
      const float m_ref = m_all == -INFINITY ? 0.f : m_all;
      float acc = 0.f, l = 0.f;
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float* src = merge + ((size_t)w * 16 + r) * STRIDE;
        const float f = exp2f(src[D] - m_ref);
        acc += src[c] * f;
        l += src[D + 1] * f;
      }
      const int row = row_start + r;
      const int token = tok0 + row / g, head = kvh * g + row % g;
      if (p.splits > 1) {
        // key splits serve tiles of ONE token: the partial sums are indexed by (tile, head)
        if (row >= g) continue;
        const size_t item = ((size_t)blockIdx.x * p.nh + head) * p.splits + split;
        p.part_acc[item * D + c] = acc;
        if (c == 0) {
          p.part_ml[item * 2] = m_all;
          p.part_ml[item * 2 + 1] = l;
        }
      } else {
        p.out[(size_t)token * p.out_stride + (size_t)head * D + c] = __float2bfloat16_rn(acc / l);
      }
    }
    if (p.splits > 1 && p.arrivals) {
      // The split that writes last merges all of them: no second kernel.  The last CTA reads the
      // others' partial results from the L2.
      __shared__ int last_to_arrive;
      __syncthreads();  // every thread's partial results are written ...
      int* counter = p.arrivals + (size_t)blockIdx.x * p.nkv + kvh;
      if (threadIdx.x == 0) {
        int ticket;  // ... and released to the GPU by the arrival itself; the last one acquires the others'
        asm volatile("atom.add.acq_rel.gpu.global.s32 %0, [%1], 1;" : "=r"(ticket) : "l"(counter) : "memory");
        last_to_arrive = ticket == my_splits - 1;
        if (last_to_arrive) *counter = 0;  // zero again for the next launch
      }
      __syncthreads();
      if (last_to_arrive) {
        // Four output elements a thread and pass.  A thread asks for every split's (max, sum) of its
        // head and for every split's four sums at once (one round trip to the L2), then weighs them.
        for (int i = threadIdx.x; i < g * (D / 4); i += THREADS) {
          const int r = i / (D / 4), c = (i % (D / 4)) * 4;
          const size_t item = ((size_t)blockIdx.x * p.nh + kvh * g + r) * p.splits;
          const float2* ml = reinterpret_cast<const float2*>(p.part_ml) + item;
          const float4* src = reinterpret_cast<const float4*>(p.part_acc + item * D + c);
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          float m_ref = -INFINITY, l = 0.f;
          for (int sp = 0; sp < my_splits; sp += 16) {
            float4 v[16];
            float2 w[16];
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const bool used = sp + j < my_splits;
              w[j] = used ? __ldcg(ml + sp + j) : make_float2(-INFINITY, 0.f);
              v[j] = used ? __ldcg(src + (size_t)(sp + j) * (D / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float m_new = m_ref;
#pragma unroll
            for (int j = 0; j < 16; ++j) m_new = fmaxf(m_new, w[j].x);
            const float m_use = m_new == -INFINITY ? 0.f : m_new;
            const float corr = exp2f(m_ref - m_use);  // 0 in the first round
            acc.x *= corr; acc.y *= corr; acc.z *= corr; acc.w *= corr;
            l *= corr;
            m_ref = m_new;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              const float f = exp2f(w[j].x - m_use);  // exp2(-inf) = 0 for the unused ones
              l = fmaf(w[j].y, f, l);
              acc.x = fmaf(v[j].x, f, acc.x);
              acc.y = fmaf(v[j].y, f, acc.y);
              acc.z = fmaf(v[j].z, f, acc.z);
              acc.w = fmaf(v[j].w, f, acc.w);
            }
          }
          const float inv = 1.f / l;
          uint2 packed;
          packed.x = pack_bf16(acc.x * inv, acc.y * inv);
          packed.y = pack_bf16(acc.z * inv, acc.w * inv);
          *reinterpret_cast<uint2*>(p.out + (size_t)tok0 * p.out_stride + (size_t)(kvh * g + r) * D + c) = packed;
        }
      }
    }
  } else {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = row_start + my_rows + (lane >> 2) + 8 * h;
      if (row >= row_end) continue;
      const int token = tok0 + row / g, head = kvh * g + row % g;
      const float inv = 1.f / l_run[h];
      __nv_bfloat16* dst = p.out + (size_t)token * p.out_stride + (size_t)head * D + (lane & 3) * 2;
#pragma unroll
      for (int i = 0; i < DTILES; ++i) {
        *reinterpret_cast<unsigned*>(dst + i * 8) = pack_bf16(o_acc[i][2 * h] * inv, o_acc[i][2 * h + 1] * inv);
      }
    }
  }
  // this grid is complete only when the one before it is: the next kernel waits for this one alone
  if (p.late_wait) tl::pdl_wait();
}

// Merges the key splits of every (decode tile, head) in a kernel of its own (used when the caller
// gives no arrival counters): one block of D threads each, thread c owning output element c.  The
// first threads turn each split's max into its weight.  Only the rows of the tiles' own tokens
// are written.
template <int D>
__global__ void __launch_bounds__(D)
attention_combine_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                         const int* __restrict__ tile_req, const int* __restrict__ req_indptr,
                         const int* __restrict__ kv_before, int window,
                         __nv_bfloat16* __restrict__ out, long long out_stride, int nh, int grid_splits) {
  tl::pdl_launch_dependents();  // the next kernel may start its prologue (it waits for us before it reads our output)
  tl::pdl_wait();               // everything before us in the stream is complete and visible

  __shared__ float weight[64];
  __shared__ float total[2];
  const int item = blockIdx.x, c = threadIdx.x;
  const int tile = item / nh, head = item % nh;
  const int req = tile_req ? tile_req[tile] : tile;
  // the splits this request used: as the attention kernel counted them
  const int hi_key = kv_before[req];
  const int lo_key = window > 0 ? max(0, hi_key - window + 1) : 0;
  const int splits = effective_splits(grid_splits, hi_key / BLOCK_N + 1 - lo_key / BLOCK_N);
  const float* ml = part_ml + (size_t)item * grid_splits * 2;
  if (c < 32) {  // splits <= 64: two per lane
    const float m0 = c < splits ? ml[2 * c] : -INFINITY;
    const float m1 = c + 32 < splits ? ml[2 * (c + 32)] : -INFINITY;
    const float m_all = tl::warp_max(fmaxf(m0, m1));
    const float m_ref = m_all == -INFINITY ? 0.f : m_all;
    const float f0 = c < splits ? exp2f(m0 - m_ref) : 0.f;
    const float f1 = c + 32 < splits ? exp2f(m1 - m_ref) : 0.f;
    weight[c] = f0;
    weight[c + 32] = f1;
    float l = (c < splits ? ml[2 * c + 1] * f0 : 0.f) + (c + 32 < splits ? ml[2 * (c + 32) + 1] * f1 : 0.f);
    l = tl::warp_sum(l);
    if (c == 0) total[0] = l;
  }
  __syncthreads();
  const float* src = part_acc + (size_t)item * grid_splits * D + c;
  float acc = 0.f;
  int s = 0;
  for (; s + 8 <= splits; s += 8) {
    float v[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = src[(size_t)(s + j) * D];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc = fmaf(v[j], weight[s + j], acc);
  }
  for (; s < splits; ++s) acc = fmaf(src[(size_t)s * D], weight[s], acc);
  const int token = req_indptr[req];
  out[(size_t)token * out_stride + (size_t)head * D + c] = __float2bfloat16_rn(acc / total[0]);
}

// Tensor maps of cache layers [rows][D] with boxes of page_size x 64 elements, by base address.
struct MapKey {
  const void* base;
  uint64_t rows;
  uint32_t cols, box_rows;
  bool operator==(const MapKey& o) const { return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows; }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return ((reinterpret_cast<size_t>(k.base) * 1000003u ^ k.rows) * 1000003u ^ k.cols) * 1000003u ^ k.box_rows;
  }
};
bool cached_map(CUtensorMap* out, const void* base, uint64_t rows, uint32_t cols, uint32_t box_rows) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex lock;
  const MapKey key{base, rows, cols, box_rows};
  std::lock_guard<std::mutex> guard(lock);
  auto it = cache.find(key);
  if (it == cache.end()) {
    CUtensorMap map;
    if (!tc_host::make_map_bf16(&map, base, rows, cols, cols, box_rows)) return false;
    if (cache.size() > 1024) cache.clear();
    it = cache.emplace(key, map).first;
  }
  *out = it->second;
  return true;
}

template <int D, bool ROWS16, bool TMA, int STAGES>
int launch(const CUtensorMap& map_kv, const Params& p, int tiles, cudaStream_t stream) {
  constexpr int BLOCK_M = ROWS16 ? 16 : 64;
  // 16-row tiles: STAGES key/value stages and Q behind them; 64-row tiles: two stages, Q inside the second.
  // TMA: room to start the stages on a 1024-byte boundary, the barriers and the abort word
  constexpr int SMEM = ((ROWS16 ? STAGES : 2) * 2 * BLOCK_N * D + (ROWS16 ? BLOCK_M * D : 0)) * 2 + (TMA ? 1024 + 64 : 0);
  static_assert(BLOCK_M * D <= 2 * BLOCK_N * D, "the Q rows fit one stage");
  static_assert(!ROWS16 || WARPS * 16 * (D + 2) * 4 <= 2 * 2 * BLOCK_N * D * 2, "merge buffer fits the stages");
  static_assert((STAGES == 2 ? 3 : 2) * (SMEM + 1024) <= 227 * 1024, "three CTAs an SM with two stages, two with three");
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attention_mma_kernel<D, ROWS16, TMA, STAGES>,
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  dim3 grid(tiles, p.nkv, p.splits);
  // Decode steps of up to 32 requests are launched overlapped with the preceding kernel:
  // the CTAs request their old key/value tiles while q is still being written.  Larger
  // grids are launched WITHOUT overlap: CTAs that start while the small kernel before them
  // still occupies the SMs are placed unevenly, and a bandwidth-bound grid's time is set by
  // its most loaded SM (measured: batch 64 decode lost 9% with an overlapped launch).
  tl::launch_kernel_opt(ROWS16 && (tiles <= p.overlap_max_tiles || p.late_wait), attention_mma_kernel<D, ROWS16, TMA, STAGES>, grid, THREADS,
                        SMEM, stream, map_kv, p);
  return TL_LAUNCH_CHECK();
}

// TORCHLET_B200_DECODE_TMA=0: the 16-row tiles gather their keys and values with cp.async (for measurements).
bool decode_tma_enabled() {
  static int value = -1;
  if (value < 0) {
    const char* v = getenv("TORCHLET_B200_DECODE_TMA");
    value = (v && atoi(v) == 0) ? 0 : 1;
  }
  return value == 1;
}

// TORCHLET_B200_DECODE_STAGES=2|3 forces the stage count of the TMA loader (for measurements).
int decode_stages() {
  static int value = -1;
  if (value < 0) {
    const char* v = getenv("TORCHLET_B200_DECODE_STAGES");
    value = v ? atoi(v) : 0;
    if (value != 2 && value != 3) value = 0;
  }
  return value;
}

template <int D>
int launch_for(const Params& p, long long num_pages, int tiles, bool rows16, cudaStream_t stream) {
  CUtensorMap map_kv;
  memset(&map_kv, 0, sizeof(map_kv));
  if (!rows16) return launch<D, false, false, 2>(map_kv, p, tiles, stream);
  const bool tma = decode_tma_enabled() && num_pages > 0 && p.page_size >= 8 && p.page_size % 8 == 0 &&
                   BLOCK_N % p.page_size == 0 &&
                   cached_map(&map_kv, p.pages, (uint64_t)num_pages * 2 * p.nkv * p.page_size, D, (uint32_t)p.page_size);
  if (!tma) return launch<D, true, false, 2>(map_kv, p, tiles, stream);
  // Without key splits (large batches) every CTA walks its request's whole context, and a third
  // stage keeps more of it requested (batch 128 at 2,048 tokens: 7.15 -> 6.68 ms a decode step;
  // batch 64: equal).  With splits the grid is sized for three CTAs an SM, which three stages do
  // not leave room for (batch 8 to 32: 5-14 % slower).
  // A grid of at most two CTAs an SM (batch 1 and 2) has the room as well: batch 1 -0.8 %.
  static int sms = 0;
  if (sms <= 0) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || sms <= 0)
      sms = 148;
  }
  const bool roomy = p.splits == 1 || (long long)tiles * p.nkv * p.splits <= 2ll * sms;
  if (decode_stages() == 3 || (decode_stages() == 0 && roomy)) return launch<D, true, true, 3>(map_kv, p, tiles, stream);
  return launch<D, true, true, 2>(map_kv, p, tiles, stream);
}

}  // namespace

TL_DEBUG_READER(tl_attention_mma_debug_error)

extern "C" {

// Bytes of float32 workspace for ``splits`` key splits of ``tiles`` decode tiles.
long long tl_attention_mma_workspace(int tiles, int nh, int d, int splits) {
  return splits > 1 ? (long long)tiles * nh * splits * (d + 2) * 4 : 0;
}

// Reads and clears the code that a bounded wait left when it gave up (0: none).
int tl_attention_mma_error() {
  int value = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&value, g_error_word, sizeof(int)) != cudaSuccess) return -1;
  if (value) cudaMemcpyToSymbol(g_error_word, &zero, sizeof(int));
  return value;
}

// rows16 != 0: tiles of 16 packed rows with the keys split over the warps and over
// ``splits`` CTAs (decode); else tiles of 64 packed rows (prompt portions), splits = 1.
// With splits > 1 every tile is a request that brings ONE token (tile_row null, at most 16
// query heads a KV head); the workspace holds tiles * nh * splits * (d + 2) floats, and only
// the output rows of those tokens are written.  ``splits`` is what the grid provides; a request
// uses as many of them as its length warrants.  ``arrivals``: tiles * nkv ints, zero before the
// call and zero again after it: the split that finishes last merges (one kernel); null: a second
// kernel merges.
// late_wait != 0 (16-row tiles only): the kernel launched just before on this stream is the prompt
// portions' attention (tl_attention_tc), which neither reads nor writes anything this call writes;
// this grid then starts beside it on the SMs it leaves idle and waits for it only at its end.
// pages: one cache layer [num_pages][2][nkv][page_size][d].
int tl_attention_mma(const void* q, long long q_stride, const void* pages, long long num_pages, const int* block_table,
                     int table_width,
                     const int* req_indptr, const int* kv_before, const int* tile_req, const int* tile_row,
                     int tiles, void* out, long long out_stride, int tokens, int nh, int nkv, int d, int page_size,
                     int window, float scale, int rows16, int splits, void* workspace, long long workspace_bytes,
                     int* arrivals, int late_wait, cudaStream_t stream) {
  if (tiles <= 0 || tokens <= 0) return 0;
  if ((d != 64 && d != 128) || nkv <= 0 || nh % nkv || page_size <= 0 || q_stride % 8 || out_stride % 4)
    return TL_ERR_UNSUPPORTED;
  if (splits < 1 || (!rows16 && splits != 1) || nkv > 65535 || splits > 64) return TL_ERR_UNSUPPORTED;
  if (splits > 1 && (tile_row || nh / nkv > 16)) return TL_ERR_UNSUPPORTED;
  if (tl_attention_mma_workspace(tiles, nh, d, splits) > workspace_bytes) return TL_ERR_UNSUPPORTED;
  Params p;
  p.q = (const __nv_bfloat16*)q;
  p.q_stride = q_stride;
  p.pages = (const __nv_bfloat16*)pages;
  p.block_table = block_table;
  p.table_width = table_width;
  p.req_indptr = req_indptr;
  p.kv_before = kv_before;
  p.tile_req = tile_req;
  p.tile_row = tile_row;
  p.out = (__nv_bfloat16*)out;
  p.out_stride = out_stride;
  p.part_acc = (float*)workspace;
  p.part_ml = p.part_acc + (size_t)tiles * nh * splits * d;
  p.arrivals = splits > 1 ? arrivals : nullptr;
  p.nh = nh;
  p.nkv = nkv;
  p.page_size = page_size;
  p.num_pages = (int)num_pages;
  p.overlap_max_tiles = 32;
  p.late_wait = (late_wait && rows16) ? 1 : 0;
  p.page_shift = -1;
  for (int b = 0; b < 20; ++b)
    if ((1 << b) == page_size) p.page_shift = b;
  p.window = window;
  p.splits = splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  const int rc = d == 128 ? launch_for<128>(p, num_pages, tiles, rows16 != 0, stream)
                           : launch_for<64>(p, num_pages, tiles, rows16 != 0, stream);
  if (rc || splits == 1 || arrivals) return rc;
  const int items = tiles * nh;
  if (d == 128)
    tl::launch_kernel(attention_combine_kernel<128>, items, 128, 0, stream, p.part_acc, p.part_ml, tile_req, req_indptr,
                      kv_before, window, p.out, out_stride, nh, splits);
  else
    tl::launch_kernel(attention_combine_kernel<64>, items, 64, 0, stream, p.part_acc, p.part_ml, tile_req, req_indptr,
                      kv_before, window, p.out, out_stride, nh, splits);
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
