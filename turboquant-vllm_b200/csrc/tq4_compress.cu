// TQ4 compress on CUDA cores (fp32 FFMA rotation): contiguous rows and the fused paged
// cache write.  One warp owns 4 rows at a time; Pi^T (pre-split into even/odd output
// columns) is staged in shared memory once per CTA and reused by every row the CTA sees.
//
// Arithmetic contract (follows the reference's PyTorch path,
// src/turboquant_vllm/quantizer.py:139-149): norm = sqrt(sum x^2) in fp32,
// xn = x / (norm + 1e-10) with IEEE division, y = xn * Pi^T with fp32 FMA accumulation in
// ascending k, idx = #{boundary < y}, byte = idx_even << 4 | idx_odd.
#include <math_constants.h>

#include "tq4_common.cuh"

namespace tq4 {

constexpr int kWarps = 8;
constexpr int kRowsPerWarp = 4;

template <int D>
struct CompressCfg {
  static constexpr int HALF = D / 2;
  static constexpr int KC = D <= 128 ? D : 64;  // k-rows of Pi^T resident in smem
  static constexpr int NCHUNK = D / KC;
  static constexpr int NBL = (HALF + 31) / 32;  // packed bytes per lane
  static constexpr int XPL = (D + 31) / 32;     // input elements per lane
  static constexpr size_t smem_bytes =
      (size_t)2 * KC * HALF * sizeof(float) + (size_t)kWarps * D * kRowsPerWarp * sizeof(float);
};

template <int D, typename T>
__global__ void __launch_bounds__(kWarps * 32)
compress_kernel(const CompressArgs a) {
  using Cfg = CompressCfg<D>;
  constexpr int HALF = Cfg::HALF, KC = Cfg::KC, NBL = Cfg::NBL, XPL = Cfg::XPL;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* s_even = reinterpret_cast<float*>(smem_raw);             // [KC][HALF]
  float* s_odd = s_even + KC * HALF;                              // [KC][HALF]
  float4* s_x = reinterpret_cast<float4*>(s_odd + KC * HALF);     // [kWarps][D] (4 rows each)

  __shared__ float s_bounds[2][16];  // ascending boundaries of each source, padded with +inf
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x < 32) {
    const int src = threadIdx.x >> 4, i = threadIdx.x & 15;
    s_bounds[src][i] = (src < a.n_sources && i < a.n_bounds[src]) ? a.bounds[src][i] : CUDART_INF_F;
  }
  float4* xw = s_x + warp * D;
  // (source, token, head) of a row; row counts fit 32 bits (checked by the host)
  const unsigned rows_per_src32 = (unsigned)(a.n_tokens * a.num_heads);
  auto row_coords = [&](int64_t row, int& src, int64_t& tok, int& h) {
    src = (uint64_t)row >= rows_per_src32 ? 1 : 0;
    const unsigned rem = (unsigned)row - (src ? rows_per_src32 : 0u);
    const unsigned t = rem / (unsigned)a.num_heads;
    tok = t;
    h = (int)(rem - t * (unsigned)a.num_heads);
  };
  const int64_t rows_per_src = a.n_tokens * a.num_heads;
  const int64_t total_rows = rows_per_src * a.n_sources;
  const int64_t n_tiles = (total_rows + kRowsPerWarp - 1) / kRowsPerWarp;
  const int64_t tiles_per_pass = (int64_t)gridDim.x * kWarps;

  auto stage_rot = [&](int chunk) {
    const float4* ge = reinterpret_cast<const float4*>(a.rot_even + (size_t)chunk * KC * HALF);
    const float4* go = reinterpret_cast<const float4*>(a.rot_odd + (size_t)chunk * KC * HALF);
    float4* se = reinterpret_cast<float4*>(s_even);
    float4* so = reinterpret_cast<float4*>(s_odd);
    for (int i = threadIdx.x; i < KC * HALF / 4; i += blockDim.x) {
      se[i] = __ldg(ge + i);
      so[i] = __ldg(go + i);
    }
  };
  if (Cfg::NCHUNK == 1) {
    stage_rot(0);
    __syncthreads();
  }

  for (int64_t pass = 0; pass * tiles_per_pass < n_tiles; ++pass) {
    const int64_t tile = pass * tiles_per_pass + (int64_t)blockIdx.x * kWarps + warp;
    const int64_t row0 = tile * kRowsPerWarp;
    float norm[kRowsPerWarp];

    // ---- load 4 rows, norm, normalise into smem --------------------------------------
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      const int64_t row = row0 + r;
      float xv[XPL];
      float ss = 0.f;
      if (row < total_rows) {
        int src, h;
        int64_t tok;
        row_coords(row, src, tok, h);
        const T* xp = reinterpret_cast<const T*>(a.x[src]) + tok * a.token_stride[src] +
                      (int64_t)h * a.head_stride[src];
#pragma unroll
        for (int i = 0; i < XPL; ++i) {
          const int k = lane + 32 * i;
          xv[i] = (k < D) ? to_float<T>(xp[k]) : 0.f;
          ss = fmaf(xv[i], xv[i], ss);
        }
      } else {
#pragma unroll
        for (int i = 0; i < XPL; ++i) xv[i] = 0.f;
      }
      ss = warp_sum(ss);
      norm[r] = sqrtf(ss);
      const float den = norm[r] + 1e-10f;
#pragma unroll
      for (int i = 0; i < XPL; ++i) {
        const int k = lane + 32 * i;
        if (k < D) reinterpret_cast<float*>(xw + k)[r] = xv[i] / den;
      }
    }
    __syncwarp();

    // ---- rotation: acc[byte][even/odd][row]; k is reduced in four quarters combined as
    //      (s0 + s1) + (s2 + s3) so the result does not depend on which kernel ran ---------
    float acc_e[NBL][kRowsPerWarp], acc_o[NBL][kRowsPerWarp];
    float t_e[NBL][kRowsPerWarp], t_o[NBL][kRowsPerWarp];   // s0 + s1, later the total
    float u_e[NBL][kRowsPerWarp], u_o[NBL][kRowsPerWarp];   // s0, later s2
    constexpr int KQ = D / 4;
#pragma unroll
    for (int i = 0; i < NBL; ++i)
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) acc_e[i][r] = acc_o[i][r] = 0.f;

    for (int chunk = 0; chunk < Cfg::NCHUNK; ++chunk) {
      if (Cfg::NCHUNK > 1) {
        __syncthreads();
        stage_rot(chunk);
        __syncthreads();
      }
#pragma unroll 4
      for (int kk = 0; kk < KC; ++kk) {
        const float4 xq = xw[chunk * KC + kk];
#pragma unroll
        for (int i = 0; i < NBL; ++i) {
          const int p = lane + 32 * i;
          const float pe = (p < HALF) ? s_even[kk * HALF + p] : 0.f;
          const float po = (p < HALF) ? s_odd[kk * HALF + p] : 0.f;
          acc_e[i][0] = fmaf(xq.x, pe, acc_e[i][0]);
          acc_e[i][1] = fmaf(xq.y, pe, acc_e[i][1]);
          acc_e[i][2] = fmaf(xq.z, pe, acc_e[i][2]);
          acc_e[i][3] = fmaf(xq.w, pe, acc_e[i][3]);
          acc_o[i][0] = fmaf(xq.x, po, acc_o[i][0]);
          acc_o[i][1] = fmaf(xq.y, po, acc_o[i][1]);
          acc_o[i][2] = fmaf(xq.z, po, acc_o[i][2]);
          acc_o[i][3] = fmaf(xq.w, po, acc_o[i][3]);
        }
        const int kg = chunk * KC + kk + 1;  // quarter boundaries (uniform branch)
        if (kg % KQ == 0) {
          const int q = kg / KQ;  // quarters finished so far
#pragma unroll
          for (int i = 0; i < NBL; ++i)
#pragma unroll
            for (int r = 0; r < kRowsPerWarp; ++r) {
              if (q == 1) { u_e[i][r] = acc_e[i][r]; u_o[i][r] = acc_o[i][r]; }
              else if (q == 2) { t_e[i][r] = u_e[i][r] + acc_e[i][r]; t_o[i][r] = u_o[i][r] + acc_o[i][r]; }
              else if (q == 3) { u_e[i][r] = acc_e[i][r]; u_o[i][r] = acc_o[i][r]; }
              else { t_e[i][r] = t_e[i][r] + (u_e[i][r] + acc_e[i][r]); t_o[i][r] = t_o[i][r] + (u_o[i][r] + acc_o[i][r]); }
              acc_e[i][r] = acc_o[i][r] = 0.f;
            }
        }
      }
    }
#pragma unroll
    for (int i = 0; i < NBL; ++i)
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) { acc_e[i][r] = t_e[i][r]; acc_o[i][r] = t_o[i][r]; }
    __syncwarp();

    // ---- bucketize, pack, store ---------------------------------------------------------
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      const int64_t row = row0 + r;
      if (row >= total_rows) continue;
      int src, h;
      int64_t tok;
      row_coords(row, src, tok, h);
      const float* b = s_bounds[src];
      uint8_t* dst_idx;
      float* dst_norm;
      if (a.cache != nullptr) {
        if (tok >= a.n_slots) continue;
        const int64_t slot = a.slot_mapping[tok];
        if (slot < 0) continue;
        if (slot >= a.num_cache_slots) {
          if (lane == 0 && a.err_flag) atomicOr(a.err_flag, TQ4_DEV_BAD_SLOT);
          continue;
        }
        const RowLayout lay = row_layout(a.num_heads, D);
        uint8_t* rowp = a.cache + slot * a.cache_token_stride;
        dst_idx = rowp + (src == 0 ? lay.k_idx : lay.v_idx) + h * HALF;
        dst_norm = reinterpret_cast<float*>(rowp + (src == 0 ? lay.k_norm : lay.v_norm) + h * 4);
      } else {
        dst_idx = a.packed_out + row * HALF;
        dst_norm = a.norms_out + row;
      }
#pragma unroll
      for (int i = 0; i < NBL; ++i) {
        const int p = lane + 32 * i;
        if (p < HALF) {
          const int ie = bucketize_sorted16(acc_e[i][r], b);
          const int io = bucketize_sorted16(acc_o[i][r], b);
          dst_idx[p] = (uint8_t)(((ie & 0xF) << 4) | (io & 0xF));
        }
      }
      if (lane == 0) *dst_norm = norm[r];
    }
    __syncwarp();
  }
}

// Small launches (decode: a few hundred to a few thousand rows): one CTA of four warps per row,
// each warp reduces one quarter of k with Pi^T read straight from L1/L2; the four partial sums
// are combined as (s0 + s1) + (s2 + s3), the same order the streaming kernel uses, so a row
// compresses to the same bytes whichever kernel handles it.
template <int D, typename T>
__global__ void __launch_bounds__(128) compress_small_kernel(const CompressArgs a) {
  using Cfg = CompressCfg<D>;
  constexpr int HALF = Cfg::HALF, NBL = Cfg::NBL, XPL = Cfg::XPL, KQ = D / 4;
  __shared__ float s_x[D];
  __shared__ float s_part[3][2 * NBL][32];
  __shared__ float s_b[16];  // ascending boundaries of this row's source, padded with +inf
  pdl_trigger();  // the query-rotation kernel that follows in a decode step does not depend on this one
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t row = blockIdx.x;
  const int64_t rows_per_src = a.n_tokens * a.num_heads;
  const int src = row >= rows_per_src ? 1 : 0;
  const unsigned rem = (unsigned)(row - (src ? rows_per_src : 0));
  const int64_t tok = rem / (unsigned)a.num_heads;
  const int h = (int)(rem - (unsigned)tok * (unsigned)a.num_heads);
  if (threadIdx.x >= 32 && threadIdx.x < 48) {
    const int i = threadIdx.x - 32;
    s_b[i] = i < a.n_bounds[src] ? a.bounds[src][i] : CUDART_INF_F;
  }
  const T* xp = reinterpret_cast<const T*>(a.x[src]) + tok * a.token_stride[src] +
                (int64_t)h * a.head_stride[src];
  float xv[XPL];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < XPL; ++i) {
    const int k = lane + 32 * i;
    xv[i] = (k < D) ? to_float<T>(xp[k]) : 0.f;
    ss = fmaf(xv[i], xv[i], ss);
  }
  ss = warp_sum(ss);
  const float norm = sqrtf(ss);
  const float den = norm + 1e-10f;
  if (warp == 0) {
#pragma unroll
    for (int i = 0; i < XPL; ++i) {
      const int k = lane + 32 * i;
      if (k < D) s_x[k] = xv[i] / den;
    }
  }
  __syncthreads();
  float acc[2 * NBL];
#pragma unroll
  for (int i = 0; i < 2 * NBL; ++i) acc[i] = 0.f;
  const int k0 = warp * KQ;
  // explicit load batches: 8 k-steps of Pi^T (up to 32 independent loads) are in flight before
  // the first FMA of the batch consumes them
  static_assert(KQ % 8 == 0, "quarter of head_dim must be a multiple of 8");
  for (int kb = 0; kb < KQ; kb += 8) {
    float pe[8][NBL], po[8][NBL];
#pragma unroll
    for (int u = 0; u < 8; ++u)
#pragma unroll
      for (int i = 0; i < NBL; ++i) {
        const int p = lane + 32 * i;
        const int k = k0 + kb + u;
        pe[u][i] = (p < HALF) ? __ldg(a.rot_even + k * HALF + p) : 0.f;
        po[u][i] = (p < HALF) ? __ldg(a.rot_odd + k * HALF + p) : 0.f;
      }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const float xk = s_x[k0 + kb + u];
#pragma unroll
      for (int i = 0; i < NBL; ++i) {
        acc[2 * i] = fmaf(xk, pe[u][i], acc[2 * i]);
        acc[2 * i + 1] = fmaf(xk, po[u][i], acc[2 * i + 1]);
      }
    }
  }
  if (warp > 0) {
#pragma unroll
    for (int i = 0; i < 2 * NBL; ++i) s_part[warp - 1][i][lane] = acc[i];
  }
  __syncthreads();
  if (warp != 0) return;
#pragma unroll
  for (int i = 0; i < 2 * NBL; ++i)
    acc[i] = (acc[i] + s_part[0][i][lane]) + (s_part[1][i][lane] + s_part[2][i][lane]);

  const float* b = s_b;
  uint8_t* dst_idx;
  float* dst_norm;
  if (a.cache != nullptr) {
    if (tok >= a.n_slots) return;
    const int64_t slot = a.slot_mapping[tok];
    if (slot < 0) return;
    if (slot >= a.num_cache_slots) {
      if (lane == 0 && a.err_flag) atomicOr(a.err_flag, TQ4_DEV_BAD_SLOT);
      return;
    }
    const RowLayout lay = row_layout(a.num_heads, D);
    uint8_t* rowp = a.cache + slot * a.cache_token_stride;
    dst_idx = rowp + (src == 0 ? lay.k_idx : lay.v_idx) + h * HALF;
    dst_norm = reinterpret_cast<float*>(rowp + (src == 0 ? lay.k_norm : lay.v_norm) + h * 4);
  } else {
    dst_idx = a.packed_out + row * HALF;
    dst_norm = a.norms_out + row;
  }
#pragma unroll
  for (int i = 0; i < NBL; ++i) {
    const int p = lane + 32 * i;
    if (p < HALF)
      dst_idx[p] =
          (uint8_t)((bucketize_sorted16(acc[2 * i], b) << 4) | bucketize_sorted16(acc[2 * i + 1], b));
  }
  if (lane == 0) *dst_norm = norm;
}


template <int D, typename T>
int launch_compress(const CompressArgs& a, cudaStream_t st) {
  using Cfg = CompressCfg<D>;
  const int64_t total_rows = a.n_tokens * a.num_heads * a.n_sources;
  if (total_rows == 0) return TQ4_OK;
  if (total_rows > 0x7fffffffll) return TQ4_ERR_INVALID_ARG;  // the kernels index rows with 32 bits
  if (total_rows <= kSmallRows) {
    compress_small_kernel<D, T><<<(unsigned)total_rows, 128, 0, st>>>(a);
    TQ4_CHECK_LAUNCH();
    return TQ4_OK;
  }
  if (!ensure_dynamic_smem<compress_kernel<D, T>>((int)Cfg::smem_bytes)) return TQ4_ERR_CUDA;
  const int64_t n_tiles = (total_rows + kRowsPerWarp - 1) / kRowsPerWarp;
  int64_t blocks = (n_tiles + kWarps - 1) / kWarps;
  const int64_t cap = (int64_t)sm_count() * 2;
  if (blocks > cap) blocks = cap;
  compress_kernel<D, T><<<(unsigned)blocks, kWarps * 32, Cfg::smem_bytes, st>>>(a);
  TQ4_CHECK_LAUNCH();
  return TQ4_OK;
}

template <int D>
int dispatch_dtype(const CompressArgs& a, int dtype, cudaStream_t st) {
  switch (dtype) {
    case TQ4_F32: return launch_compress<D, float>(a, st);
    case TQ4_F16: return launch_compress<D, __half>(a, st);
    case TQ4_BF16: return launch_compress<D, __nv_bfloat16>(a, st);
  }
  return TQ4_ERR_UNSUPPORTED;
}

int dispatch_compress(const CompressArgs& a, int head_dim, int dtype, cudaStream_t st) {
  if (a.n_tokens * a.num_heads * a.n_sources > kSmallRows) {
    if (compress_tc16_eligible(a, head_dim, dtype)) return launch_compress_tc16(a, dtype, st);
    if (compress_tc_eligible(a, head_dim, dtype)) return launch_compress_tc(a, dtype, st);
  }
  switch (head_dim) {
    case 64: return dispatch_dtype<64>(a, dtype, st);
    case 96: return dispatch_dtype<96>(a, dtype, st);
    case 128: return dispatch_dtype<128>(a, dtype, st);
    case 256: return dispatch_dtype<256>(a, dtype, st);
  }
  return TQ4_ERR_UNSUPPORTED;
}

// bucketize + pack pre-rotated rows: one thread per packed byte.
__global__ void pack_rotated_kernel(const float* __restrict__ y, int64_t n_rows, int half,
                                    const float* __restrict__ b, int nb,
                                    uint8_t* __restrict__ out) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_rows * half) return;
  const float2 v = reinterpret_cast<const float2*>(y)[i];
  out[i] = (uint8_t)((bucketize(v.x, b, nb) << 4) | bucketize(v.y, b, nb));
}

}  // namespace tq4

extern "C" int tq4_compress_rows(const void* x, int x_dtype, int64_t n_tokens, int num_heads,
                                 int head_dim, int64_t x_token_stride, int64_t x_head_stride,
                                 const float* rot_t_even, const float* rot_t_odd,
                                 const float* boundaries, int n_boundaries,
                                 uint8_t* packed_out, float* norms_out, void* stream) {
  if (n_tokens < 0 || num_heads <= 0) return TQ4_ERR_INVALID_ARG;
  if (!tq4::supported_head_dim(head_dim)) return TQ4_ERR_UNSUPPORTED;
  if (n_boundaries < 0 || n_boundaries > TQ4_MAX_BOUNDARIES) return TQ4_ERR_UNSUPPORTED;
  if (n_tokens == 0) return TQ4_OK;
  if (!x || !rot_t_even || !rot_t_odd || !boundaries || !packed_out || !norms_out)
    return TQ4_ERR_INVALID_ARG;
  if (((uintptr_t)rot_t_even | (uintptr_t)rot_t_odd) & 15) return TQ4_ERR_INVALID_ARG;
  tq4::CompressArgs a{};
  a.x[0] = x;
  a.token_stride[0] = x_token_stride;
  a.head_stride[0] = x_head_stride;
  a.bounds[0] = boundaries;
  a.n_bounds[0] = n_boundaries;
  a.n_tokens = n_tokens;
  a.num_heads = num_heads;
  a.n_sources = 1;
  a.rot_even = rot_t_even;
  a.rot_odd = rot_t_odd;
  a.packed_out = packed_out;
  a.norms_out = norms_out;
  tq4::prof_begin(TQ4_PROF_COMPRESS, (cudaStream_t)stream);
  a.x_dtype = x_dtype;
  const int rc = tq4::dispatch_compress(a, head_dim, x_dtype, (cudaStream_t)stream);
  tq4::prof_end(TQ4_PROF_COMPRESS, (cudaStream_t)stream);
  return rc;
}

extern "C" int tq4_pack_rotated_rows(const float* rotated, int64_t n_rows, int head_dim,
                                     const float* boundaries, int n_boundaries,
                                     uint8_t* packed_out, void* stream) {
  if (n_rows < 0 || head_dim <= 0 || (head_dim & 1)) return TQ4_ERR_INVALID_ARG;
  if (n_boundaries < 0 || n_boundaries > TQ4_MAX_BOUNDARIES) return TQ4_ERR_UNSUPPORTED;
  if (n_rows == 0) return TQ4_OK;
  if (!rotated || !boundaries || !packed_out || ((uintptr_t)rotated & 7)) return TQ4_ERR_INVALID_ARG;
  const int64_t n = n_rows * (head_dim / 2);
  tq4::pack_rotated_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
      rotated, n_rows, head_dim / 2, boundaries, n_boundaries, packed_out);
  TQ4_CHECK_LAUNCH();
  return TQ4_OK;
}

extern "C" int tq4_write_paged(const void* key, const void* value, int kv_dtype,
                               int64_t n_tokens, int num_kv_heads, int head_dim,
                               int64_t k_token_stride, int64_t k_head_stride,
                               int64_t v_token_stride, int64_t v_head_stride,
                               const int64_t* slot_mapping, int64_t n_slots,
                               const float* rot_t_even, const float* rot_t_odd,
                               const float* k_boundaries, int n_k_boundaries,
                               const float* v_boundaries, int n_v_boundaries,
                               uint8_t* cache, int64_t cache_token_stride, int64_t num_cache_slots,
                               int* err_flag, void* stream) {
  if (n_tokens < 0 || n_slots < 0 || num_kv_heads <= 0) return TQ4_ERR_INVALID_ARG;
  if (!tq4::supported_head_dim(head_dim)) return TQ4_ERR_UNSUPPORTED;
  if (n_k_boundaries < 0 || n_k_boundaries > TQ4_MAX_BOUNDARIES || n_v_boundaries < 0 ||
      n_v_boundaries > TQ4_MAX_BOUNDARIES)
    return TQ4_ERR_UNSUPPORTED;
  if (n_tokens == 0 || n_slots == 0) return TQ4_OK;
  if (!key || !value || !slot_mapping || !rot_t_even || !rot_t_odd || !k_boundaries ||
      !v_boundaries || !cache)
    return TQ4_ERR_INVALID_ARG;
  if (((uintptr_t)rot_t_even | (uintptr_t)rot_t_odd) & 15) return TQ4_ERR_INVALID_ARG;
  if (((uintptr_t)cache & 3) || (cache_token_stride & 3) ||
      cache_token_stride < tq4::row_data_bytes(num_kv_heads, head_dim))
    return TQ4_ERR_INVALID_ARG;
  tq4::CompressArgs a{};
  a.x[0] = key;
  a.x[1] = value;
  a.token_stride[0] = k_token_stride;
  a.head_stride[0] = k_head_stride;
  a.token_stride[1] = v_token_stride;
  a.head_stride[1] = v_head_stride;
  a.bounds[0] = k_boundaries;
  a.n_bounds[0] = n_k_boundaries;
  a.bounds[1] = v_boundaries;
  a.n_bounds[1] = n_v_boundaries;
  a.n_tokens = n_tokens < n_slots ? n_tokens : n_slots;
  a.num_heads = num_kv_heads;
  a.n_sources = 2;
  a.rot_even = rot_t_even;
  a.rot_odd = rot_t_odd;
  a.cache = cache;
  a.slot_mapping = slot_mapping;
  a.n_slots = n_slots;
  a.cache_token_stride = cache_token_stride;
  a.num_cache_slots = num_cache_slots;
  a.err_flag = err_flag;
  tq4::prof_begin(TQ4_PROF_WRITE, (cudaStream_t)stream);
  a.x_dtype = kv_dtype;
  const int rc = tq4::dispatch_compress(a, head_dim, kv_dtype, (cudaStream_t)stream);
  tq4::prof_end(TQ4_PROF_WRITE, (cudaStream_t)stream);
  return rc;
}
