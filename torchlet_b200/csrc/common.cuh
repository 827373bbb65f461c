// Shared helpers of the hand-written sm_100a kernels.
//
// Every launcher is an extern "C" function that takes raw device pointers, sizes
// and a CUDA stream, launches on that stream and returns the cudaError_t of the
// launch as an int (0 = success).  Element types are passed as codes:
//   0 = float32, 1 = bfloat16.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define TL_DTYPE_F32 0
#define TL_DTYPE_BF16 1

// Returned by launchers for arguments a kernel refuses (never a wrong result).
#define TL_ERR_UNSUPPORTED 10001

#define TL_LAUNCH_CHECK() ((int)cudaGetLastError())

// ------------------------------------------------------------------ debug build
// Built with -DTL_DEBUG (environment: TORCHLET_B200_DEBUG=1) the kernels check the indices they
// are handed before they use them: a token id against the vocabulary, a position against the
// width of its block table, a page id against the pool, a slot against the slot range.  A check
// that fails records (code, offending value) in the library's two debug words -- the first
// failure wins -- and the kernel SKIPS the access, so nothing faults; the host reads the words
// with the library's tl_<name>_debug_error() and raises.  (The stand-in for a memory checker on
// machines where none may run.)  Without the flag the checks cost nothing.
#define TL_DEBUG_TOKEN 1     // token id outside [0, vocabulary)
#define TL_DEBUG_POSITION 2  // position beyond the request's block table
#define TL_DEBUG_PAGE 3      // page id outside [0, pages in the pool)
#define TL_DEBUG_SLOT 4      // slot outside [0, slots)
#ifdef TL_DEBUG
__device__ int g_tl_debug_words[2] = {0, 0};
#define TL_DEBUG_OK(condition, code, value) tl_debug_ok((condition), (code), (int)(value))
__device__ __forceinline__ bool tl_debug_ok(bool condition, int code, int value) {
  if (!condition && atomicCAS(&g_tl_debug_words[0], 0, code) == 0) g_tl_debug_words[1] = value;
  return condition;
}
// Defines the library's reader: returns the code (0: none) and stores the value; reading clears.
#define TL_DEBUG_READER(name)                                                                       \
  extern "C" int name(int* value) {                                                                 \
    int words[2] = {0, 0}, zero[2] = {0, 0};                                                        \
    if (cudaMemcpyFromSymbol(words, g_tl_debug_words, sizeof(words)) != cudaSuccess) return -1;     \
    if (words[0]) cudaMemcpyToSymbol(g_tl_debug_words, zero, sizeof(zero));                         \
    if (value) *value = words[1];                                                                   \
    return words[0];                                                                                \
  }
#else
#define TL_DEBUG_OK(condition, code, value) true
#define TL_DEBUG_READER(name)             \
  extern "C" int name(int* value) {       \
    if (value) *value = 0;                \
    return 0;                             \
  }
#endif

#include <stdlib.h>

namespace tl {

// ---------------------------------------------------- programmatic dependent launch
// Kernels are launched with the programmatic-stream-serialization attribute: a kernel
// may START while its predecessor in the stream is still running, once every CTA of the
// predecessor has executed pdl_launch_dependents() (or exited).  It must execute
// pdl_wait() before it touches anything an earlier kernel wrote or still reads; the wait
// returns when the predecessor has completed and its memory operations are visible.
// Work that depends on no earlier kernel (barrier set-up, streaming weights) may come
// before the wait and so overlaps the predecessor's tail.  Every kernel here executes
// pdl_wait() in every CTA, so completion of a kernel implies completion of all before it.
// TORCHLET_B200_PDL=0 in the environment launches everything fully serialized.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

inline bool pdl_enabled() {
  static int enabled = -1;
  if (enabled < 0) {
    const char* v = getenv("TORCHLET_B200_PDL");
    enabled = (v && v[0] == '0') ? 0 : 1;
  }
  return enabled == 1;
}

// ``overlap`` false: this launch waits for the full completion of its predecessor.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_opt(bool overlap, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                     cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = (overlap && pdl_enabled()) ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = smem;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = pdl_enabled() ? 1 : 0;
  return cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of NT threads (NT a multiple of 32, at most 1024); every thread
// gets the result.  The order of additions depends only on NT.
template <int NT> __device__ __forceinline__ float block_sum(float v, float* scratch /*[32]*/) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  float t = (lane < NT / 32) ? scratch[lane] : 0.f;
  return warp_sum(t);
}

// 8 consecutive elements as floats (pointer 16- or 32-byte aligned by construction).
__device__ __forceinline__ void load8(const float* p, float (&out)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p);
  const float4 b = *reinterpret_cast<const float4*>(p + 4);
  out[0] = a.x; out[1] = a.y; out[2] = a.z; out[3] = a.w;
  out[4] = b.x; out[5] = b.y; out[6] = b.z; out[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float (&out)[8]) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}

}  // namespace tl
