// TQ4 decompress (rotated space): unpack nibbles, centroid LUT, scale by the fp32 norm,
// cast.  One thread expands one 32-bit word of packed indices (8 coordinates) and stores
// them with a single 16- or 32-byte write.
#include "tq4_common.cuh"

namespace tq4 {

template <typename T>
struct alignas(sizeof(T) * 8 > 16 ? 16 : sizeof(T) * 8) Vec8 {
  T v[8];
};

template <typename T>
__device__ __forceinline__ void expand_word(uint32_t w, float norm, const float* lut, T* dst) {
  Vec8<T> o;
#pragma unroll
  for (int b = 0; b < 4; ++b) {
    const uint32_t byte = (w >> (8 * b)) & 0xFFu;
    o.v[2 * b] = from_float<T>(lut[byte >> 4] * norm);
    o.v[2 * b + 1] = from_float<T>(lut[byte & 0xFu] * norm);
  }
  *reinterpret_cast<Vec8<T>*>(dst) = o;
}

template <typename T>
__global__ void decompress_rows_kernel(const uint8_t* __restrict__ packed,
                                       const float* __restrict__ norms,
                                       const float* __restrict__ centroids, int n_cent,
                                       int64_t n_rows, int words_per_row, T* __restrict__ out) {
  __shared__ float lut[TQ4_MAX_CENTROIDS];
  if (threadIdx.x < TQ4_MAX_CENTROIDS)
    lut[threadIdx.x] = threadIdx.x < n_cent ? centroids[threadIdx.x] : 0.f;
  __syncthreads();
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_rows * words_per_row) return;
  const int64_t row = i / words_per_row;
  const uint32_t w = reinterpret_cast<const uint32_t*>(packed)[i];
  expand_word<T>(w, norms[row], lut, out + i * 8);
}

// Token rows of a paged cache -> K and V [n_slots, H, D].
template <typename T>
__global__ void decompress_cache_kernel(const uint8_t* __restrict__ cache, int64_t token_stride,
                                        int64_t n_slots, int H, int D,
                                        const float* __restrict__ k_cent, int n_k,
                                        const float* __restrict__ v_cent, int n_v,
                                        T* __restrict__ k_out, T* __restrict__ v_out) {
  __shared__ float lut[2][TQ4_MAX_CENTROIDS];
  if (threadIdx.x < TQ4_MAX_CENTROIDS) {
    lut[0][threadIdx.x] = threadIdx.x < n_k ? k_cent[threadIdx.x] : 0.f;
    lut[1][threadIdx.x] = threadIdx.x < n_v ? v_cent[threadIdx.x] : 0.f;
  }
  __syncthreads();
  const int wpr = D / 8;  // words per (token, head)
  const int64_t per_src = n_slots * H * wpr;
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= 2 * per_src) return;
  const int src = (int)(i / per_src);
  const int64_t j = i - (int64_t)src * per_src;
  const int64_t th = j / wpr;  // token*H + head
  const int wi = (int)(j - th * wpr);
  const int64_t tok = th / H;
  const int h = (int)(th - tok * H);
  const RowLayout lay = row_layout(H, D);
  const uint8_t* row = cache + tok * token_stride;
  const uint32_t w = *reinterpret_cast<const uint32_t*>(row + (src ? lay.v_idx : lay.k_idx) +
                                                        h * (D / 2) + wi * 4);
  const float norm = *reinterpret_cast<const float*>(row + (src ? lay.v_norm : lay.k_norm) + h * 4);
  expand_word<T>(w, norm, lut[src], (src ? v_out : k_out) + j * 8);
}

}  // namespace tq4

extern "C" int tq4_decompress_rows(const uint8_t* packed, const float* norms,
                                   const float* centroids, int n_centroids, int64_t n_rows,
                                   int head_dim, void* out, int out_dtype, void* stream) {
  if (n_rows < 0 || head_dim <= 0 || head_dim % 8) return TQ4_ERR_UNSUPPORTED;
  if (n_centroids <= 0 || n_centroids > TQ4_MAX_CENTROIDS) return TQ4_ERR_UNSUPPORTED;
  if (n_rows == 0) return TQ4_OK;
  if (!packed || !norms || !centroids || !out) return TQ4_ERR_INVALID_ARG;
  if (((uintptr_t)packed & 3) || ((uintptr_t)out & 15)) return TQ4_ERR_INVALID_ARG;
  const int wpr = head_dim / 8;
  const int64_t n = n_rows * wpr;
  const unsigned grid = (unsigned)((n + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
  switch (out_dtype) {
    case TQ4_F32:
      tq4::decompress_rows_kernel<float><<<grid, 256, 0, st>>>(packed, norms, centroids, n_centroids,
                                                               n_rows, wpr, (float*)out);
      break;
    case TQ4_F16:
      tq4::decompress_rows_kernel<__half><<<grid, 256, 0, st>>>(packed, norms, centroids, n_centroids,
                                                                n_rows, wpr, (__half*)out);
      break;
    case TQ4_BF16:
      tq4::decompress_rows_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
          packed, norms, centroids, n_centroids, n_rows, wpr, (__nv_bfloat16*)out);
      break;
    default:
      return TQ4_ERR_UNSUPPORTED;
  }
  TQ4_CHECK_LAUNCH();
  return TQ4_OK;
}

extern "C" int tq4_decompress_cache(const uint8_t* cache, int64_t cache_token_stride,
                                    int64_t n_slots, int num_kv_heads, int head_dim,
                                    const float* k_centroids, int n_k_centroids,
                                    const float* v_centroids, int n_v_centroids,
                                    void* k_out, void* v_out, int out_dtype, void* stream) {
  if (n_slots < 0 || num_kv_heads <= 0 || head_dim <= 0 || head_dim % 8) return TQ4_ERR_UNSUPPORTED;
  if (n_k_centroids <= 0 || n_k_centroids > TQ4_MAX_CENTROIDS || n_v_centroids <= 0 ||
      n_v_centroids > TQ4_MAX_CENTROIDS)
    return TQ4_ERR_UNSUPPORTED;
  if (n_slots == 0) return TQ4_OK;
  if (!cache || !k_centroids || !v_centroids || !k_out || !v_out) return TQ4_ERR_INVALID_ARG;
  if (((uintptr_t)cache & 3) || (cache_token_stride & 3) || ((uintptr_t)k_out & 15) ||
      ((uintptr_t)v_out & 15) ||
      cache_token_stride < tq4::row_data_bytes(num_kv_heads, head_dim))
    return TQ4_ERR_INVALID_ARG;
  const int64_t n = 2 * n_slots * num_kv_heads * (head_dim / 8);
  const unsigned grid = (unsigned)((n + 255) / 256);
  cudaStream_t st = (cudaStream_t)stream;
  switch (out_dtype) {
    case TQ4_F32:
      tq4::decompress_cache_kernel<float><<<grid, 256, 0, st>>>(
          cache, cache_token_stride, n_slots, num_kv_heads, head_dim, k_centroids, n_k_centroids,
          v_centroids, n_v_centroids, (float*)k_out, (float*)v_out);
      break;
    case TQ4_F16:
      tq4::decompress_cache_kernel<__half><<<grid, 256, 0, st>>>(
          cache, cache_token_stride, n_slots, num_kv_heads, head_dim, k_centroids, n_k_centroids,
          v_centroids, n_v_centroids, (__half*)k_out, (__half*)v_out);
      break;
    case TQ4_BF16:
      tq4::decompress_cache_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
          cache, cache_token_stride, n_slots, num_kv_heads, head_dim, k_centroids, n_k_centroids,
          v_centroids, n_v_centroids, (__nv_bfloat16*)k_out, (__nv_bfloat16*)v_out);
      break;
    default:
      return TQ4_ERR_UNSUPPORTED;
  }
  TQ4_CHECK_LAUNCH();
  return TQ4_OK;
}
