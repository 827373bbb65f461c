// The per-request slot records on the device, and the two kernels that stand at the two ends of
// a captured decode step.
//
// A slot is the stable index a live request keeps (the reference's decode slots,
// v05_decode_slots/scheduler.py:38-71, with static per-slot buffers for token, position and
// activity, v06_static_buffers/scheduler.py:42-52).  Here a slot's record lives on the device:
//
//   records[0][s]  last token        records[3][s]  temperature (float bits)
//   records[1][s]  position = cached tokens so far  records[4..5][s]  seed (low, high word)
//   records[2][s]  tokens sampled so far (the generator's counter)
//
// and so do the block tables of all slots, slot_tables[group][slot][width].  A decode step that is
// replayed from a CUDA graph reads its lanes' tokens, positions, sampling words and table rows
// from these records (slot_gather), and advances them itself when it has sampled (slot_advance):
// position + 1, counter + 1, token = the sampled one.  The host therefore sends, a step, only a
// small command block: which slot stands in which lane, the records of lanes that are new in the
// decode set (or whose token the caller supplies), and the table entries that were added.
#include "common.cuh"

namespace {

constexpr int RECORD_ROWS = 6;

// command block (int32 words):
//   [0] live lanes   [1] number of table entries
//   lanes[b]   slot of each lane, -1: padding
//   flags[b]   bit 0: take position, counter, temperature, seed from the block; bit 1: take the token
//   token[b] position[b] counter[b] temperature[b] seed_low[b] seed_high[b]
//   entries[2 * capacity]   (index into slot_tables, page) pairs
__global__ void __launch_bounds__(128)
slot_gather_kernel(const int* __restrict__ command, int b, int groups, int max_slots, int width, int page_size,
                   int* __restrict__ records, int* __restrict__ slot_tables, int* __restrict__ lane_token,
                   int* __restrict__ lane_position, int* __restrict__ lane_kv_before, int* __restrict__ lane_slot,
                   long long* __restrict__ lane_seed, float* __restrict__ lane_temperature,
                   int* __restrict__ lane_counter, int* __restrict__ lane_tables) {
  // No early start for the next kernel: some kernels of the step read the lane words this kernel
  // writes before their own wait (the decode attention plans its key tiles from them), which is
  // sound only if every kernel after this one starts after this one has ended.
  tl::pdl_wait();  // the command block's copy and everything before it are complete
  const int lane = blockIdx.x, tid = threadIdx.x;
  const int entries = command[1];
  const int* lanes = command + 2;
  const int* flags = lanes + b;
  const int* given = flags + b;  // six rows of b words
  const int* pairs = given + 6 * b;
  const int slot = lanes[lane];
  TL_DEBUG_OK(slot >= -1 && slot < max_slots, TL_DEBUG_SLOT, slot);  // -1 is the padding mark
  if (slot < 0 || slot >= max_slots) {  // padding: token 0 at position 0 of the reserved page 0
    if (tid == 0) {
      lane_token[lane] = 0;
      lane_position[lane] = 0;
      lane_kv_before[lane] = 0;
      lane_slot[lane] = 0;
      lane_seed[lane] = 0;
      lane_temperature[lane] = 0.f;
      lane_counter[lane] = 0;
    }
    if (tid < groups) lane_tables[((size_t)tid * b + lane) * width] = 0;
    return;
  }
  // table entries added since the slot's last step (each lane takes those of its own slot)
  for (int i = tid; i < entries; i += blockDim.x) {
    const int index = pairs[2 * i];
    if ((index / width) % max_slots == slot) slot_tables[index] = pairs[2 * i + 1];
  }
  if (tid == 0) {
    const int f = flags[lane];
    if (f & 1) {
      records[1 * max_slots + slot] = given[1 * b + lane];
      records[2 * max_slots + slot] = given[2 * b + lane];
      records[3 * max_slots + slot] = given[3 * b + lane];
      records[4 * max_slots + slot] = given[4 * b + lane];
      records[5 * max_slots + slot] = given[5 * b + lane];
    }
    if (f & 2) records[0 * max_slots + slot] = given[0 * b + lane];
  }
  __syncthreads();
  const int position = records[1 * max_slots + slot];
  TL_DEBUG_OK(position >= 0 && position / page_size < width, TL_DEBUG_POSITION, position);
  if (tid == 0) {
    lane_token[lane] = records[0 * max_slots + slot];
    lane_position[lane] = position;
    lane_kv_before[lane] = position;
    lane_slot[lane] = slot;
    lane_counter[lane] = records[2 * max_slots + slot];
    lane_temperature[lane] = __int_as_float(records[3 * max_slots + slot]);
    const unsigned long long low = (unsigned)records[4 * max_slots + slot], high = (unsigned)records[5 * max_slots + slot];
    lane_seed[lane] = (long long)(low | (high << 32));
  }
  // the slot's table rows, as far as the step reads them: the pages up to the new token's
  const int used = min(width, position / page_size + 1);
  for (int g = 0; g < groups; ++g) {
    const int* src = slot_tables + ((size_t)g * max_slots + slot) * width;
    int* dst = lane_tables + ((size_t)g * b + lane) * width;
    for (int i = tid; i < used; i += blockDim.x) dst[i] = src[i];
  }
}

__global__ void slot_advance_kernel(const int* __restrict__ command, int b, int max_slots,
                                    const int* __restrict__ sampled, int* __restrict__ records) {
  tl::pdl_wait();
  tl::pdl_launch_dependents();
  const int lane = blockIdx.x * blockDim.x + threadIdx.x;
  if (lane >= b) return;
  const int slot = command[2 + lane];
  if (slot < 0 || slot >= max_slots) return;
  records[0 * max_slots + slot] = sampled[lane];
  records[1 * max_slots + slot] += 1;
  records[2 * max_slots + slot] += 1;
}

}  // namespace

TL_DEBUG_READER(tl_slots_debug_error)

extern "C" {

int tl_slot_record_rows() { return RECORD_ROWS; }

// Words of the command block of a step of ``b`` lanes with room for ``capacity`` table entries.
int tl_slot_command_words(int b, int capacity) { return 2 + 8 * b + 2 * capacity; }

int tl_slot_gather(const int* command, int b, int groups, int max_slots, int width, int page_size, int* records,
                   int* slot_tables, int* lane_token, int* lane_position, int* lane_kv_before, int* lane_slot,
                   long long* lane_seed, float* lane_temperature, int* lane_counter, int* lane_tables,
                   cudaStream_t stream) {
  if (b <= 0) return 0;
  if (groups < 0 || groups > 128 || max_slots <= 0 || width <= 0 || page_size <= 0) return TL_ERR_UNSUPPORTED;
  tl::launch_kernel(slot_gather_kernel, b, 128, 0, stream, command, b, groups, max_slots, width, page_size, records,
                    slot_tables, lane_token, lane_position, lane_kv_before, lane_slot, lane_seed, lane_temperature,
                    lane_counter, lane_tables);
  return TL_LAUNCH_CHECK();
}

int tl_slot_advance(const int* command, int b, int max_slots, const int* sampled, int* records, cudaStream_t stream) {
  if (b <= 0) return 0;
  tl::launch_kernel(slot_advance_kernel, (b + 127) / 128, 128, 0, stream, command, b, max_slots, sampled, records);
  return TL_LAUNCH_CHECK();
}

}  // extern "C"
