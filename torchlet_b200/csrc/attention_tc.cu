// Paged causal grouped-query attention for PROMPT PORTIONS on the 5th-generation tensor
// cores (tcgen05), bfloat16, head_dim 64 or 128 (a template parameter: an operand tile is one
// or two 64-element slabs wide).
//
// One CTA takes two tiles of up to 128 PACKED ROWS of one (request, KV head): the pairs
// (token of the step, query head of the KV head's group), token-major, so every key/value
// tile that is loaded serves all query heads of the group and both row tiles.  It walks
// over the keys in tiles of 128 absolute positions:
//
//   loader warps    one for K, one for V: TMA-load the tile's pages (one box of page_size x 64
//                   elements per page and 64-element slab of the head, 128-byte swizzle, one
//                   lane per box) through the block table into a two-stage ring;
//   MMA warp        for each row tile X in turn:  O_X += P_X V of the previous key tile
//                   (P_X read from tensor memory, V as the MN-major operand from shared
//                   memory), then S_X = Q_X K^T of this key tile (Q and K K-major in shared
//                   memory).  S_X, P_X (in the first half of S_X's columns) and O_X live
//                   in tensor memory: 2 x 128 + 2 x head_dim columns (all 512 for head_dim 128);
//   softmax warps   four warps per row tile, one thread per row: read the row of S from
//                   tensor memory, mask by position, keep the running max and sum in
//                   float32, write P as bfloat16 over S, and rescale O in tensor memory
//                   when the row's max has grown by more than 2^8 since O was last scaled
//                   (a smaller growth is carried in P, whose exponent range has room for
//                   it).  While one row tile is in its softmax the tensor core works for
//                   the other.
//
// The tensor core executes one thread's MMAs in the order of issue, so S_X of the next key
// tile, issued after P_X V of this one, cannot overwrite P_X early, and O_X is at rest
// whenever S_X has arrived (the arrival covers the P_X V before it).
//
// At the end the softmax warps divide O by the row sums and store bfloat16 output.
// Numerics are those of attention_mma.cu and of the reference's Triton kernel
// (v10_triton_paged_gqa/kernel/gqa.py:91-111): float32 scores scaled by head_dim^-0.5,
// float32 max/sum/accumulator, P rounded to the value dtype before P V.
//
// Every mbarrier wait is bounded (tcgen05.cuh); a wait that gives up records a code that
// tl_attention_tc_error() returns, and the CTA still runs to its end and frees its TMEM.
#include <math.h>
#include <string.h>

#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "tcgen05.cuh"

namespace {

using namespace tc;

constexpr int ROWS = 128;       // packed rows of a row tile (UMMA M)
constexpr int QTILES = 2;       // row tiles a CTA
constexpr int KEYS = 128;       // keys a tile (UMMA N of S, K of P V)
constexpr int THREADS = 352;    // warps 0-3 softmax of row tile 0, 4-7 of row tile 1, 8 MMA, 9 and 10 loaders
constexpr int SLAB = ROWS * 128;  // bytes of a [128 rows][64 bf16] swizzled slab
// a 128 x D bf16 operand tile = D / 64 slabs
template <int D> struct TileBytes { static constexpr int value = (D / 64) * SLAB; };
constexpr float RESCALE_THRESHOLD = 8.f;  // log2 units

__device__ int g_error_word = 0;

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
  int splits;       // CTAs (blockIdx.z) that share the key tiles of one (row tiles, KV head)
  float* part_acc;  // splits > 1: [tokens * nh][splits][D] unnormalized outputs
  float* part_ml;   //             [tokens * nh][splits][2] reference max (log2 units) and sum
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
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Instruction descriptor for O += P V: A (P) K-major, B (V) MN-major (bit 16).
template <int D> __device__ __forceinline__ uint32_t idesc_pv() { return idesc_bf16_f32(ROWS, D) | (1u << 16); }

// Shared-memory descriptor of the MN-major operand V: a tile is one or two slabs (64 elements
// of the head each) of [128 keys][64 elements]; 8 keys form a 1024-byte swizzle atom (stride
// byte offset), the slabs are SLAB bytes apart (leading byte offset).
__device__ __forceinline__ uint64_t smem_desc_v(uint32_t saddr) {
  uint64_t desc = 0;
  desc |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  desc |= (uint64_t)(SLAB >> 4) << 16;
  desc |= (uint64_t)(1024 >> 4) << 32;
  desc |= (uint64_t)1 << 46;
  desc |= (uint64_t)2 << 61;
  return desc;
}

// D (+)= A B with A read from tensor memory: row i of A in lane i, two bfloat16 of
// consecutive k in each 32-bit column (16 k = 8 columns an instruction).
__device__ __forceinline__ void mma_bf16_a_tmem(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                                bool accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}\n" ::"r"(tmem_d),
      "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
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

// P = exp2(S * scale - m) of one row as bfloat16 pairs into tensor memory at ``tmem_p`` (64
// columns).  The row's sum of the unrounded P goes to sum_a + sum_b.
__device__ __forceinline__ void exp_and_store(const uint32_t (&v)[KEYS], float scale_log2, float neg_m, uint32_t tmem_p,
                                              float& sum_a, float& sum_b) {
#pragma unroll
  for (int c = 0; c < KEYS; c += 64) {
    uint32_t packed[32];
#pragma unroll
    for (int i = 0; i < 64; i += 2) {
      const float xa = fmaf(__uint_as_float(v[c + i]), scale_log2, neg_m);
      const float xb = fmaf(__uint_as_float(v[c + i + 1]), scale_log2, neg_m);
      const float a = fast_exp2(xa), b = fast_exp2(xb);
      sum_a += a;
      sum_b += b;
      __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
      packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
    }
    tmem_st_32(tmem_p + (c >> 1), packed);
  }
}

// Key tiles [begin, end) that row tile X of the CTA needs; rows [row_start, row_end).
struct RowTile {
  int row_start, row_end, begin, end;
};

template <int D>
__global__ void __launch_bounds__(THREADS, 1)
attention_tc_kernel(const __grid_constant__ CUtensorMap map_kv, const Params p) {
  constexpr int TILE_BYTES = TileBytes<D>::value;
  constexpr int SLABS = D / 64;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_tiles = smem;                      // 2 row tiles
  uint8_t* k_tiles = smem + 2 * TILE_BYTES;     // 2 stages
  uint8_t* v_tiles = smem + 4 * TILE_BYTES;     // 2 stages
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + 6 * TILE_BYTES);
  uint64_t* k_full = bars;        // [2 stages]
  uint64_t* v_full = bars + 2;    // [2 stages]
  uint64_t* k_empty = bars + 4;   // [2 stages]
  uint64_t* v_empty = bars + 6;   // [2 stages]
  uint64_t* s_full = bars + 8;    // [2 row tiles]  S_X of the next key tile is in tensor memory
  uint64_t* p_full = bars + 10;   // [2 row tiles]  (4 arrivals: one per softmax warp) P_X is written
  uint64_t* o_done = bars + 12;   // [2 row tiles]  the last P_X V is done
  uint64_t* v_clean = bars + 14;  // value rows outside the CTA's keys are cleared (edge tiles only)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // KV heads vary fastest over the grid: the CTAs of the row tiles that see the most keys (the
  // caller lists those first) start first for ALL heads, and the short ones fill the end
  const int kvh = blockIdx.x;
  const int req = p.tile_req[blockIdx.y];
  const int g = p.nh / p.nkv;
  const int tok0 = p.req_indptr[req];
  const int q_len = p.req_indptr[req + 1] - tok0;
  const int before = p.kv_before[req];
  const int* table = p.block_table + (size_t)req * p.table_width;
  RowTile tile[QTILES];
  int cta_lo_key = 0, cta_hi_key = -1;  // the keys any row of the CTA may see
#pragma unroll
  for (int x = 0; x < QTILES; ++x) {
    RowTile& t = tile[x];
    t.row_start = p.tile_row[blockIdx.y] + x * p.rows_per_tile;
    t.row_end = min(q_len * g, t.row_start + p.rows_per_tile);
    t.begin = t.end = 0;
    if (t.row_start < t.row_end) {
      const int first_tok = t.row_start / g, last_tok = (t.row_end - 1) / g;
      const int lo_key = p.window > 0 ? max(0, before + first_tok - p.window + 1) : 0;
      t.begin = lo_key / KEYS;
      t.end = (before + last_tok) / KEYS + 1;
      if (x == 0) cta_lo_key = lo_key;
      cta_hi_key = before + last_tok;
    }
  }
  // Later rows need later keys, so the row tiles' key tiles are [first of tile 0, last of the last tile)
  const int all_begin = tile[0].begin;
  const int all_end = max(tile[0].end, tile[1].end);
  // With key splits (a small grid: few row tiles for the whole GPU) this CTA takes its share of
  // them and leaves partial results for the merge kernel.
  int j_begin = all_begin, j_end = all_end;
  const int split = blockIdx.z;
  if (p.splits > 1) {
    const int per = (all_end - all_begin + p.splits - 1) / p.splits;
    j_begin = min(all_end, all_begin + split * per);
    j_end = min(all_end, j_begin + per);
#pragma unroll
    for (int x = 0; x < QTILES; ++x) {
      tile[x].begin = min(max(tile[x].begin, j_begin), j_end);
      tile[x].end = max(min(tile[x].end, j_end), tile[x].begin);
    }
  }
  // Whole pages are copied, so the first and the last key tile may hold rows of keys outside
  // [cta_lo_key, cta_hi_key]: whatever the pages held before.  Their weights are exactly 0, but
  // 0 x NaN is NaN, so the V loader clears those value rows before the tensor core reads them.
  const bool edge_first = cta_lo_key % KEYS != 0 && j_begin == all_begin && j_begin < j_end;
  const bool edge_last = cta_hi_key % KEYS != KEYS - 1 && j_end == all_end && j_begin < j_end;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 4);
      mbar_init(&o_done[i], 1);
    }
    mbar_init(v_clean, 1);
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tensormap(&map_kv);
  }
  if (warp == 8) {
    tmem_alloc<512>(tmem_slot);
    tmem_relinquish();
  }
  // First the wait, then the signal: when the next kernel starts, every CTA of this one has seen
  // the preceding kernels' q, keys and values complete.  A decode attention launched right behind
  // may therefore start on the SMs this grid leaves idle without a wait of its own at its start
  // (csrc/attention_mma.cu, ``late_wait``).
  tl::pdl_wait();
  tl::pdl_launch_dependents();

  // ---- Q rows into shared memory in the K-major swizzled layout (all threads)
  for (int i = threadIdx.x; i < QTILES * ROWS * (D / 8); i += THREADS) {
    const int x = i / (ROWS * (D / 8)), r = (i / (D / 8)) % ROWS, c16 = i % (D / 8);
    const int row = (x == 0 ? tile[0].row_start : tile[1].row_start) + r;
    const bool valid = r < p.rows_per_tile && row < (x == 0 ? tile[0].row_end : tile[1].row_end);
    const __nv_bfloat16* src = p.q;
    if (valid) src = p.q + (size_t)(tok0 + row / g) * p.q_stride + (size_t)(kvh * g + row % g) * D + c16 * 8;
    uint8_t* dst = q_tiles + x * TILE_BYTES + (c16 >> 3) * SLAB + r * 128 + (((c16 & 7) ^ (r & 7)) << 4);
    cp_async_16(dst, src, valid);
  }
  asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory");
  fence_proxy_async();  // the tensor core reads what ordinary stores and cp.async wrote
  fence_before_sync();
  __syncthreads();
  fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= 9) {
    // ----------------------------------------------------------------- loaders
    // Warp 9 copies K, warp 10 copies V.  Lane l copies slab (l % SLABS) of page (l / SLABS) of
    // every tile: a box of page_size keys x 64 elements (page_size >= 8, so a tile has at most 16
    // pages).  The copies of a tile cost their issue, not their bytes: thirty-two issued by
    // one thread take longer than the tile's arithmetic.
    const int is_v = warp - 9;
    uint8_t* tiles = is_v ? v_tiles : k_tiles;
    uint64_t* full = is_v ? v_full : k_full;
    uint64_t* empty = is_v ? v_empty : k_empty;
    const int pages_per_tile = KEYS / p.page_size;
    const int my_page = lane / SLABS, my_half = lane % SLABS;
    const bool active = my_page < pages_per_tile;
    for (int j = j_begin; j < j_end; ++j) {
      const int jj = j - j_begin, s = jj & 1;
      const uint32_t phase = (jj >> 1) & 1;
      const int index = j * pages_per_tile + my_page;
      const int page = (active && index < p.table_width) ? table[index] : 0;  // beyond the table: page 0
      const uint32_t offset = s * TILE_BYTES + my_half * SLAB + my_page * p.page_size * 128;
      mbar_wait(&empty[s], phase ^ 1, abort_flag, &g_error_word, 1 + is_v);
      if (lane == 0) mbar_expect_tx(&full[s], TILE_BYTES);
      __syncwarp();
      if (active)
        tma_load_2d(tiles + offset, &map_kv, &full[s], my_half * 64, ((page * 2 + is_v) * p.nkv + kvh) * p.page_size);
      if (is_v && ((edge_first && j == j_begin) || (edge_last && j == j_end - 1))) {
        mbar_wait(&full[s], phase, abort_flag, &g_error_word, 10);  // the tile has landed
        for (int i = lane; i < KEYS * SLABS * 8; i += 32) {  // a key's row: 128 bytes in each slab
          const int k = i / (SLABS * 8), key = j * KEYS + k;
          if (key < cta_lo_key || key > cta_hi_key)
            *reinterpret_cast<uint4*>(tiles + s * TILE_BYTES + ((i >> 3) % SLABS) * SLAB + k * 128 + (i & 7) * 16) =
                make_uint4(0u, 0u, 0u, 0u);
        }
        fence_proxy_async();  // the tensor core reads, and later copies overwrite, what these stores wrote
        __syncwarp();
        if (lane == 0) mbar_arrive(v_clean);
      }
    }
  } else if (warp == 8) {
    // --------------------------------------------------------------------- MMA
    // The whole warp walks the loop and waits; one elected lane issues (with the loop inside a
    // one-lane branch the operands of every MMA went through per-lane registers, and issuing
    // took longer than the MMAs run).  The tensor core's queue is short, and every wait, fence
    // and election costs the warp tens of nanoseconds in which it issues nothing, while eight
    // of these MMAs run for 280 ns: so a row tile's P V and next S go out together, behind one
    // wait for its P.  The tiles take turns, which keeps one in its softmax while the other's
    // MMAs run.
    const uint32_t idesc_s = idesc_bf16_f32(ROWS, KEYS);
    const uint32_t idesc_o = idesc_pv<D>();
    // Descriptors of the operands' first 16-wide slices; a later slice adds its byte offset / 16
    // to the address field (the tiles lie below 256 KB, so the field never carries).
    const uint64_t q_desc[QTILES] = {smem_desc_sw128(smem_addr(q_tiles)), smem_desc_sw128(smem_addr(q_tiles + TILE_BYTES))};
    const uint64_t k_desc[2] = {smem_desc_sw128(smem_addr(k_tiles)), smem_desc_sw128(smem_addr(k_tiles + TILE_BYTES))};
    const uint64_t v_desc[2] = {smem_desc_v(smem_addr(v_tiles)), smem_desc_v(smem_addr(v_tiles + TILE_BYTES))};
    // One step past the last key tile, for the P V that runs a tile behind
    for (int j = j_begin; j <= j_end; ++j) {
      const int jj = j - j_begin;
      // V of the previous key tile has long arrived, K of this one nearly always
      if (jj > 0) mbar_wait(&v_full[(jj - 1) & 1], ((jj - 1) >> 1) & 1, abort_flag, &g_error_word, 6);
      if (jj > 0 && ((edge_first && j - 1 == j_begin) || (edge_last && j == j_end)))
        mbar_wait(v_clean, (edge_first && edge_last && j == j_end && j_end - j_begin > 1) ? 1 : 0, abort_flag,
                  &g_error_word, 11);
      if (j < j_end) mbar_wait(&k_full[jj & 1], (jj >> 1) & 1, abort_flag, &g_error_word, 3);
      // the last row tile with work at this step (row tile 0 always has some)
      const bool work_1 = (j - 1 >= tile[1].begin && j - 1 < tile[1].end) || (j >= tile[1].begin && j < tile[1].end);
#pragma unroll
      for (int x = 0; x < QTILES; ++x) {
        const uint32_t tmem_s = tmem_base + x * KEYS;     // S_x, and P_x in its first 64 columns
        const uint32_t tmem_o = tmem_base + 256 + x * D;  // O_x
        const bool do_pv = j - 1 >= tile[x].begin && j - 1 < tile[x].end;  // O_x (+)= P_x V of key tile j - 1
        const bool do_s = j >= tile[x].begin && j < tile[x].end;           // S_x = Q_x K^T of key tile j
        if (!do_pv && !do_s) continue;
        const int t = j - 1 - tile[x].begin;
        if (do_pv) mbar_wait(&p_full[x], t & 1, abort_flag, &g_error_word, 5);
        fence_after_sync();
        if (elect_one()) {
          if (do_pv) {
            const uint64_t b_desc = ((jj - 1) & 1) ? v_desc[1] : v_desc[0];
#pragma unroll
            for (int k = 0; k < KEYS / 16; ++k)  // 16 keys: 8 columns of P, two 8-key atoms of V (2048 bytes)
              mma_bf16_a_tmem(tmem_o, tmem_s + k * 8, b_desc + (uint64_t)(k * (2048 >> 4)), idesc_o, t > 0 || k > 0);
            if (j == tile[x].end) mma_commit(&o_done[x]);
          }
          if (do_s) {
            const uint64_t b_desc = (jj & 1) ? k_desc[1] : k_desc[0];
#pragma unroll
            for (int k = 0; k < D / 16; ++k) {  // slab k / 4, 32 bytes a slice within its 128-byte rows
              const uint64_t offset = (uint64_t)(((k >> 2) * SLAB + (k & 3) * 32) >> 4);
              mma_bf16(tmem_s, q_desc[x] + offset, b_desc + offset, idesc_s, k > 0);
            }
            mma_commit(&s_full[x]);
          }
          // The warp's MMAs are all issued by the lane that elect.sync names, the same every
          // time, so its commits cover them
          if (x == 1 || !work_1) {
            if (j < j_end) mma_commit(&k_empty[jj & 1]);
            if (jj > 0) mma_commit(&v_empty[(jj - 1) & 1]);
          }
        }
        __syncwarp();
      }
    }
  } else {
    // ----------------------------------------------------------------- softmax
    const int x = warp >> 2, quarter = warp & 3;
    const RowTile mine = x == 0 ? tile[0] : tile[1];
    const int r = quarter * 32 + lane;  // row of the tile = lane of tensor memory
    const int row = mine.row_start + r;
    const bool row_valid = r < p.rows_per_tile && row < mine.row_end;
    const int pos = row_valid ? before + row / g : -1;
    const int lo = (row_valid && p.window > 0) ? max(0, pos - p.window + 1) : 0;
    const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
    const uint32_t tmem_s = tmem_base + x * KEYS + lane_base;
    const uint32_t tmem_o = tmem_base + 256 + x * D + lane_base;
    const int num_tiles = mine.end - mine.begin;
    float m_ref = -INFINITY, l_sum = 0.f;  // m_ref in log2 units (already scaled)
    for (int t = 0; t < num_tiles; ++t) {
      const int key0 = (mine.begin + t) * KEYS;
      mbar_wait(&s_full[x], t & 1, abort_flag, &g_error_word, 7);
      fence_after_sync();
      uint32_t v[KEYS];  // the row of S, in registers
#pragma unroll
      for (int c = 0; c < KEYS; c += 32) tmem_ld_32(tmem_s + c, reinterpret_cast<uint32_t(&)[32]>(v[c]));
      tmem_ld_wait();
      // A tile whose keys are all visible to every row of this warp needs no masking; rows beyond
      // the tile's last (zero queries, never stored) take whatever comes
      const bool visible = !row_valid || (key0 + KEYS - 1 <= pos && key0 >= lo);
      const bool all_visible = __all_sync(0xffffffffu, visible);
      if (!all_visible) {
        const int first_rel = lo - key0;
        const unsigned span = row_valid ? (unsigned)(pos - lo) : 0x7fffffffu;
#pragma unroll
        for (int i = 0; i < KEYS; ++i) {
          // key0 + i outside [lo, pos], as one unsigned comparison
          if ((unsigned)(i - first_rel) > span) v[i] = __float_as_uint(-INFINITY);
        }
      }
      float m_a = -INFINITY, m_b = -INFINITY, m_c = -INFINITY, m_d = -INFINITY;
#pragma unroll
      for (int i = 0; i < KEYS; i += 8) {
        m_a = max3(m_a, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
        m_b = max3(m_b, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
        m_c = max3(m_c, __uint_as_float(v[i + 4]), __uint_as_float(v[i + 5]));
        m_d = max3(m_d, __uint_as_float(v[i + 6]), __uint_as_float(v[i + 7]));
      }
      const float m_tile = fmaxf(fmaxf(m_a, m_b), fmaxf(m_c, m_d)) * p.scale_log2;  // the scale is positive
      // the reference max moves only when the row's max has grown past the threshold
      float factor = 1.f;
      bool rescale = false;
      if (m_tile > m_ref + RESCALE_THRESHOLD || (m_ref == -INFINITY && m_tile > -INFINITY)) {
        factor = m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - m_tile);
        rescale = m_ref != -INFINITY;
        m_ref = m_tile;
      }
      l_sum *= factor;
      if (__any_sync(0xffffffffu, rescale)) {
        // O_x is at rest: the arrival of S_x covered the P_x V issued before it
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t o[32];
          tmem_ld_32(tmem_o + c, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
          tmem_st_32(tmem_o + c, o);
        }
      }
      // P = exp2(S * scale - m_ref) as bfloat16 pairs over the first half of S's columns; row sum
      const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
      float sum_a = 0.f, sum_b = 0.f;
      exp_and_store(v, p.scale_log2, neg_m, tmem_s, sum_a, sum_b);
      l_sum += sum_a + sum_b;
      tmem_st_wait();
      fence_before_sync();  // our tcgen05.ld/st of S, P and O are done
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[x]);
    }
    // ---- output.  With key splits: the unnormalized O with its reference max and sum, for the merge
    if (p.splits > 1) {
      const size_t item = row_valid ? ((size_t)(tok0 + row / g) * p.nh + kvh * g + row % g) * p.splits + split : 0;
      if (num_tiles > 0) {
        mbar_wait(&o_done[x], 0, abort_flag, &g_error_word, 9);
        fence_after_sync();
        float* dst = p.part_acc + item * D;
#pragma unroll 1
        for (int c = 0; c < D; c += 32) {
          uint32_t o[32];
          tmem_ld_32(tmem_o + c, o);
          tmem_ld_wait();
          if (row_valid) {
#pragma unroll
            for (int q4 = 0; q4 < 8; ++q4)
              *reinterpret_cast<uint4*>(dst + c + 4 * q4) = make_uint4(o[4 * q4], o[4 * q4 + 1], o[4 * q4 + 2], o[4 * q4 + 3]);
          }
        }
      }
      if (row_valid) {  // a split that saw no key of this row says so: the merge leaves its O alone
        p.part_ml[item * 2] = num_tiles > 0 ? m_ref : -INFINITY;
        p.part_ml[item * 2 + 1] = num_tiles > 0 ? l_sum : 0.f;
      }
    } else if (num_tiles > 0) {
      mbar_wait(&o_done[x], 0, abort_flag, &g_error_word, 9);
      fence_after_sync();
      const float inv = l_sum > 0.f ? 1.f / l_sum : 0.f;
      __nv_bfloat16* dst = nullptr;
      if (row_valid) dst = p.out + (size_t)(tok0 + row / g) * p.out_stride + (size_t)(kvh * g + row % g) * D;
#pragma unroll 1
      for (int c = 0; c < D; c += 32) {
        uint32_t o[32];
        tmem_ld_32(tmem_o + c, o);
        tmem_ld_wait();
        if (row_valid) {
          uint32_t packed[16];
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
            packed[i >> 1] = *reinterpret_cast<uint32_t*>(&h);
          }
#pragma unroll
          for (int q4 = 0; q4 < 4; ++q4)
            *reinterpret_cast<uint4*>(dst + c + 8 * q4) =
                make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
        }
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

// Merges the key splits of every (token, head) of the requests that brought more than one token:
// out = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M).  One warp an item; a lane owns D / 32 elements.
template <int D>
__global__ void __launch_bounds__(128)
attention_tc_merge_kernel(const float* __restrict__ part_acc, const float* __restrict__ part_ml,
                          const int* __restrict__ token_req, const int* __restrict__ req_indptr,
                          __nv_bfloat16* __restrict__ out, long long out_stride, int tokens, int nh, int splits) {
  tl::pdl_launch_dependents();
  tl::pdl_wait();
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= tokens * nh) return;
  const int token = item / nh, head = item % nh;
  const int req = token_req[token];
  if (req_indptr[req + 1] - req_indptr[req] < 2) return;  // a single token: the decode kernel's row
  const float* ml = part_ml + (size_t)item * splits * 2;
  float m_all = -INFINITY;
  for (int s = 0; s < splits; ++s) m_all = fmaxf(m_all, ml[2 * s]);
  constexpr int PER = D / 32;
  float acc[PER], total = 0.f;
#pragma unroll
  for (int i = 0; i < PER; ++i) acc[i] = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float m = ml[2 * s];
    if (m == -INFINITY) continue;  // that split saw no key of this row and wrote no O
    const float f = exp2f(m - m_all);
    total = fmaf(ml[2 * s + 1], f, total);
    const float* src = part_acc + ((size_t)item * splits + s) * D + lane * PER;
#pragma unroll
    for (int i = 0; i < PER; ++i) acc[i] = fmaf(src[i], f, acc[i]);
  }
  const float inv = total > 0.f ? 1.f / total : 0.f;
  __nv_bfloat16* dst = out + (size_t)token * out_stride + (size_t)head * D + lane * PER;
#pragma unroll
  for (int i = 0; i < PER; ++i) dst[i] = __float2bfloat16_rn(acc[i] * inv);
}

// ------------------------------------------------------------------ host side
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

template <int D>
int launch_merge(const Params& p, const int* token_req, int tokens, cudaStream_t stream) {
  tl::launch_kernel(attention_tc_merge_kernel<D>, (tokens * p.nh + 3) / 4, 128, 0, stream, (const float*)p.part_acc,
                    (const float*)p.part_ml, token_req, p.req_indptr, p.out, p.out_stride, tokens, p.nh, p.splits);
  return TL_LAUNCH_CHECK();
}

template <int D>
int launch(const CUtensorMap& map_kv, const Params& p, int nkv, int tiles, const int* token_req, int tokens,
           bool defer_merge, cudaStream_t stream) {
  constexpr int SMEM = 6 * TileBytes<D>::value + 1024 + 256;
  static_assert(SMEM <= 232448, "shared memory of one CTA");
  static bool configured = false;
  if (!configured) {
    cudaError_t err = cudaFuncSetAttribute(attention_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (err != cudaSuccess) return (int)err;
    configured = true;
  }
  tl::launch_kernel(attention_tc_kernel<D>, dim3(nkv, tiles, p.splits), THREADS, SMEM, stream, map_kv, p);
  const int rc = TL_LAUNCH_CHECK();
  if (rc || p.splits == 1 || defer_merge) return rc;
  return launch_merge<D>(p, token_req, tokens, stream);
}

}  // namespace

extern "C" {

int tl_attention_tc_error() {
  int value = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&value, g_error_word, sizeof(int)) != cudaSuccess) return -1;
  if (value) cudaMemcpyToSymbol(g_error_word, &zero, sizeof(int));
  return value;
}

// Packed rows a CTA takes for a group of ``group`` query heads: two row tiles of whole tokens.
int tl_attention_tc_rows(int group) { return group > 0 && group <= ROWS ? QTILES * (ROWS / group) * group : 0; }

// Bytes of float32 workspace for ``splits`` key splits over the ``tokens`` tokens of a step.
long long tl_attention_tc_workspace(int tokens, int nh, int d, int splits) {
  return splits > 1 ? (long long)tokens * nh * splits * (d + 2) * 4 : 0;
}

// pages: one cache layer [num_pages][2][nkv][page_size][d] bf16, d 64 or 128.  tile_req / tile_row:
// request and first packed row (a multiple of tl_attention_tc_rows(nh / nkv)) of each CTA; the
// tiles cover every request of the step that brings more than one token.
// splits > 1 (for grids that would leave most of the GPU idle): that many CTAs share the key
// tiles of each (row tiles, KV head) and a second kernel merges their partial results, which
// live in ``workspace`` (tl_attention_tc_workspace bytes); token_req [tokens] names each token's
// request.  defer_merge != 0: the merge is left to a later tl_attention_tc_merge on the same stream
// (so that another kernel may run between the two; the workspace must stay untouched meanwhile).
int tl_attention_tc(const void* q, long long q_stride, const void* pages, long long num_pages,
                    const int* block_table, int table_width, const int* req_indptr, const int* kv_before,
                    const int* tile_req, const int* tile_row, int tiles, void* out, long long out_stride, int nh,
                    int nkv, int d, int page_size, int window, float scale, int splits, const int* token_req,
                    int tokens, void* workspace, long long workspace_bytes, int defer_merge, cudaStream_t stream) {
  if (tiles <= 0) return 0;
  if (splits < 1 || splits > 64) return TL_ERR_UNSUPPORTED;
  if (splits > 1 && (!token_req || tokens <= 0 || !workspace ||
                     workspace_bytes < tl_attention_tc_workspace(tokens, nh, d, splits)))
    return TL_ERR_UNSUPPORTED;
  if ((d != 64 && d != 128) || nkv <= 0 || nh % nkv || nh / nkv > ROWS || page_size < 8 || page_size > KEYS ||
      KEYS % page_size || q_stride % 8 || out_stride % 8 || tiles > 65535 || !tile_req || !tile_row)
    return TL_ERR_UNSUPPORTED;
  CUtensorMap map_kv;
  if (!cached_map(&map_kv, pages, (uint64_t)num_pages * 2 * nkv * page_size, (uint32_t)d, (uint32_t)page_size))
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
  p.rows_per_tile = tl_attention_tc_rows(nh / nkv) / QTILES;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.splits = splits;
  p.part_acc = (float*)workspace;
  p.part_ml = p.part_acc + (size_t)(splits > 1 ? tokens : 0) * nh * splits * d;
  return d == 128 ? launch<128>(map_kv, p, nkv, tiles, token_req, tokens, defer_merge != 0, stream)
                  : launch<64>(map_kv, p, nkv, tiles, token_req, tokens, defer_merge != 0, stream);
}

// The merge that a tl_attention_tc call with defer_merge left undone: same out, sizes, splits,
// token_req and workspace as that call.
int tl_attention_tc_merge(const int* req_indptr, void* out, long long out_stride, int nh, int d, int splits,
                          const int* token_req, int tokens, void* workspace, long long workspace_bytes,
                          cudaStream_t stream) {
  if (splits <= 1 || tokens <= 0) return 0;
  if ((d != 64 && d != 128) || !token_req || !workspace || out_stride % 8 ||
      workspace_bytes < tl_attention_tc_workspace(tokens, nh, d, splits))
    return TL_ERR_UNSUPPORTED;
  Params p;
  memset(&p, 0, sizeof(p));
  p.req_indptr = req_indptr;
  p.out = (__nv_bfloat16*)out;
  p.out_stride = out_stride;
  p.nh = nh;
  p.splits = splits;
  p.part_acc = (float*)workspace;
  p.part_ml = p.part_acc + (size_t)tokens * nh * splits * d;
  return d == 128 ? launch_merge<128>(p, token_req, tokens, stream) : launch_merge<64>(p, token_req, tokens, stream);
}

}  // extern "C"
