// Shared device/host helpers for the TQ4 sm_100a kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tq4.h"

#define TQ4_MAX_BOUNDARIES 15
#define TQ4_MAX_CENTROIDS 16

#define TQ4_CHECK_LAUNCH()                                   \
  do {                                                       \
    cudaError_t e__ = cudaGetLastError();                    \
    if (e__ != cudaSuccess) return (int)TQ4_ERR_CUDA;        \
  } while (0)

namespace tq4 {

// per-kernel event timing (tq4_profile.cu); no-ops unless tq4_profile_start() was called
void prof_begin(int kind, cudaStream_t st);
void prof_end(int kind, cudaStream_t st);

// ---- programmatic dependent launch ---------------------------------------------------------------
// The kernels of one decode step (cache write, query rotation + plan, attention, merge) are launched
// back to back.  A kernel that calls pdl_trigger() lets the next launch in the stream start before it
// has finished, if that launch was made with launch_kernel(..., pdl = true); the dependent kernel
// calls pdl_wait() before it reads or writes anything a predecessor touches: after the wait, the
// preceding kernel has completed and its stores are visible.  Rules kept by every kernel here:
//  * the FIRST kernel an entry point launches is a plain stream-ordered launch (pdl = false): its
//    inputs may come from the caller's preceding kernel, which may itself trigger dependents early;
//  * the later kernels of the same entry point are launched with pdl = true; before pdl_wait() they
//    only read caller inputs (which the first kernel's launch has already ordered behind the
//    caller's work) and write shared memory or registers;
//  * a kernel launched with pdl = true calls pdl_wait() on every path before it exits, so its own
//    completion implies the completion of everything before it in the stream.
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
bool pdl_enabled();  // false if TQ4_NO_PDL is set in the environment

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                 cudaStream_t st, bool pdl, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = (pdl && pdl_enabled()) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__host__ __device__ inline bool supported_head_dim(int d) {
  return d == 64 || d == 96 || d == 128 || d == 256;
}

// Bytes of one token row that carry data: [K_idx|K_norm|V_idx|V_norm].
__host__ __device__ inline int row_data_bytes(int num_kv_heads, int head_dim) {
  return num_kv_heads * (head_dim + 8);
}

struct RowLayout {
  int k_idx, k_norm, v_idx, v_norm;  // byte offsets of the four regions in a token row
};
__host__ __device__ inline RowLayout row_layout(int num_kv_heads, int head_dim) {
  RowLayout r;
  r.k_idx = 0;
  r.k_norm = num_kv_heads * (head_dim / 2);
  r.v_idx = r.k_norm + num_kv_heads * 4;
  r.v_norm = r.v_idx + num_kv_heads * (head_dim / 2);
  return r;
}

template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Load one element of a typed tensor chosen at run time (cold paths only).
__device__ __forceinline__ float load_as_float(const void* p, int dtype, int64_t i) {
  if (dtype == TQ4_F32) return reinterpret_cast<const float*>(p)[i];
  if (dtype == TQ4_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void store_from_float(void* p, int dtype, int64_t i, float v) {
  if (dtype == TQ4_F32) reinterpret_cast<float*>(p)[i] = v;
  else if (dtype == TQ4_F16) reinterpret_cast<__half*>(p)[i] = __float2half_rn(v);
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
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

// idx = #{b : b < y}: the tie rule of torch.bucketize(right=False).  NaN compares false -> 0.
__device__ __forceinline__ int bucketize(float y, const float* __restrict__ b, int nb) {
  int idx = 0;
#pragma unroll
  for (int i = 0; i < TQ4_MAX_BOUNDARIES; ++i)
    if (i < nb) idx += (y > b[i]) ? 1 : 0;
  return idx;
}

// The same count by binary search over ASCENDING boundaries padded to 15 entries with +inf
// (entry 15 is never read): four compares.  NaN compares false at every step -> 0.
__device__ __forceinline__ int bucketize_sorted16(float y, const float* b) {
  int lo = (y > b[7]) ? 8 : 0;
  lo += (y > b[lo + 3]) ? 4 : 0;
  lo += (y > b[lo + 1]) ? 2 : 0;
  lo += (y > b[lo]) ? 1 : 0;
  return lo;
}

// address of element i of an array of dtype-coded elements
__device__ __forceinline__ const void* byte_offset(const void* p, int dtype, int64_t i) {
  return reinterpret_cast<const char*>(p) + i * (dtype == TQ4_F32 ? 4 : 2);
}

// out[i][v] = element 32*i of the strip starting at base[v] (nullptr -> zeros), converted to fp32
template <typename T, int N, int V>
__device__ __forceinline__ void load_strip(const void* const (&base)[V], float (&out)[N][V]) {
#pragma unroll
  for (int v = 0; v < V; ++v)
#pragma unroll
    for (int i = 0; i < N; ++i)
      out[i][v] = base[v] ? to_float<T>(reinterpret_cast<const T*>(base[v])[32 * i]) : 0.f;
}

// ---- per-device host state ---------------------------------------------------------------------
// A process may drive several GPUs (a model spread over devices, one thread per GPU).  Function
// attributes set with cudaFuncSetAttribute and device properties belong to ONE device, so
// everything remembered on the host side is indexed by the ordinal of the current device.
constexpr int kMaxDevices = 64;
inline int device_ordinal() {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -1;
  return dev;
}

inline int sm_count() {
  static int n[kMaxDevices];
  const int dev = device_ordinal();
  if (dev < 0) return 148;
  if (n[dev] == 0) {
    cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev);
    if (n[dev] <= 0) n[dev] = 148;
  }
  return n[dev];
}

// Opt `Kernel` in to `bytes` of dynamic shared memory on the current device (once per device and
// kernel; again if a later call asks for more).
template <auto Kernel>
inline bool ensure_dynamic_smem(int bytes, bool max_carveout = false) {
  static int set_bytes[kMaxDevices];
  const int dev = device_ordinal();
  if (dev < 0) return false;
  if (set_bytes[dev] >= bytes && set_bytes[dev] > 0) return true;
  if (cudaFuncSetAttribute(Kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess)
    return false;
  if (max_carveout)
    cudaFuncSetAttribute(Kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  set_bytes[dev] = bytes;
  return true;
}

// Arguments of the compress / cache-write kernels (tq4_compress.cu) and of the write part of the
// fused prologue kernel (tq4_attention.cu).
struct CompressArgs {
  // sources: [0] = K (or the only tensor), [1] = V (paged write only)
  const void* x[2];
  int64_t token_stride[2], head_stride[2];
  const float* bounds[2];
  int n_bounds[2];
  int64_t n_tokens;
  int num_heads;
  int n_sources;  // 1 or 2
  int x_dtype;    // TQ4_F32 / TQ4_F16 / TQ4_BF16 of both sources (read by the fused prologue kernel)
  const float* rot_even;
  const float* rot_odd;
  // contiguous destination
  uint8_t* packed_out;
  float* norms_out;
  // paged destination (cache != nullptr selects it)
  uint8_t* cache;
  const int64_t* slot_mapping;
  int64_t n_slots, cache_token_stride, num_cache_slots;
  int* err_flag;
};

// rows at or below this count are handled by the small-launch kernels
constexpr int64_t kSmallRows = 8192;
int dispatch_compress(const CompressArgs& a, int head_dim, int dtype, cudaStream_t st);
// tensor-core (tcgen05) compress kernel for large inputs at head_dim 128 (tq4_compress_tc.cu)
bool compress_tc_eligible(const CompressArgs& a, int head_dim, int dtype);
int launch_compress_tc(const CompressArgs& a, int dtype, cudaStream_t st);
// pipelined tcgen05 kernel for dense 16-bit inputs at head_dim 128 (tq4_compress_tc16.cu)
bool compress_tc16_eligible(const CompressArgs& a, int head_dim, int dtype);
int launch_compress_tc16(const CompressArgs& a, int dtype, cudaStream_t st);

}  // namespace tq4
