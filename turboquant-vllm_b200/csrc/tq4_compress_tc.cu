// TQ4 compress for prefill-sized inputs at head_dim 128 on the 5th-generation tensor cores:
// the rotation y = x^ * Pi^T of a tile of 128 vectors is a 128 x 128 x 128 GEMM issued as
// tcgen05.mma (kind::tf32) with the accumulator in tensor memory.
//
// Precision.  TF32 keeps 10 mantissa bits, so each fp32 operand is split into hi + lo with
// hi = the top 19 bits of the value and lo = value - hi (exact in fp32), and the product is
// accumulated as hi*hi + hi*lo + lo*hi in fp32: the dropped lo*lo term and the bits of lo beyond
// TF32 are below 2^-20 of |x||Pi|.  A rotated coordinate therefore differs from the fp32 FMA
// kernels by ~1e-7 absolute, which moves an index only when the coordinate sits that close to a
// bucket boundary (measured mismatch ~1e-5 of the indices, bound 1e-4).  Norms are computed in the
// exact order of the FMA kernels (lane-strided FMAs, butterfly tree), so they are bit-identical.
//
// Data flow per tile (one persistent CTA per SM, 256 threads; thread = (row, half of the columns)):
//   norm of the row (both threads of a row, redundantly)                      CUDA cores
//   x^ = x * (1 / (norm + 1e-10)), split, stored K-major with the 128-byte swizzle   CUDA cores -> smem
//   48 x tcgen05.mma 128x128x8 over two K-steps of 64, D in 128 TMEM columns   tensor cores
//   tcgen05.ld of the thread's 64 columns, bucketize, pack, store              CUDA cores
// Pi (hi and lo) stays resident in shared memory: 2 x 64 KB.  Every wait is bounded.
#include <cuda.h>
#include <math_constants.h>

#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "tq4_common.cuh"

namespace tq4 {
namespace {

constexpr int kD = 128;               // head_dim handled here
constexpr int kRows = 128;            // vectors per tile (MMA M, TMEM lanes)
constexpr int kThreads = 256;
constexpr int kBlockBytes = kRows * 128;         // one K-block (32 tf32 columns) of an operand: 16 KB
constexpr uint32_t kOffBhi = 0, kOffBlo = 4 * kBlockBytes, kOffA = 8 * kBlockBytes;
constexpr uint32_t kSmemBytes = 8 * kBlockBytes + 2 * 2 * kBlockBytes;  // Pi hi/lo + two A buffers (hi, lo)
constexpr uint32_t kOffX = kSmemBytes;            // XT: the tile's 128 input rows (16-bit), two column halves
constexpr uint32_t kXBytes = 2 * kBlockBytes;     // 2 x [128 rows][64 elements = 128 B], 128-byte swizzle
constexpr uint32_t kTmemCols = 128;
// instruction descriptor: D = F32, A = B = TF32, both K-major, N = 128, M = 128
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// shared-memory matrix descriptor: K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);  // start address / 16
  d |= (uint64_t)1 << 16;                    // leading byte offset (unused for swizzled K-major)
  d |= (uint64_t)(1024 >> 4) << 32;          // stride byte offset between 8-row groups
  d |= (uint64_t)1 << 46;                    // descriptor version of this architecture
  d |= (uint64_t)2 << 61;                    // SWIZZLE_128B
  return d;
}
// byte offset of (row, 16-byte chunk c of the row's 128 bytes) inside a K-block
__device__ __forceinline__ uint32_t swz(int row, int c) { return (uint32_t)(row * 128 + ((c ^ (row & 7)) << 4)); }

__device__ __forceinline__ bool elect_one_sync() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo) {
  hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
  lo = x - hi;
}

__device__ __forceinline__ void mma_tf32(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(kInstrDesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool bar_wait_bounded(uint32_t bar, uint32_t parity) {
  for (int it = 0; it < (1 << 22); ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
  }
  return false;
}

template <typename T>
struct RowLoader;  // 32 consecutive elements of a row -> fp32
template <>
struct RowLoader<float> {
  static __device__ __forceinline__ void load32(const float* p, float (&x)[32]) {
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(p) + i);
      x[4 * i] = v.x; x[4 * i + 1] = v.y; x[4 * i + 2] = v.z; x[4 * i + 3] = v.w;
    }
  }
};
template <>
struct RowLoader<__half> {
  static __device__ __forceinline__ void load32(const __half* p, float (&x)[32]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(p) + i);
      const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __half22float2(h[j]);
        x[8 * i + 2 * j] = f.x; x[8 * i + 2 * j + 1] = f.y;
      }
    }
  }
};
template <>
struct RowLoader<__nv_bfloat16> {
  static __device__ __forceinline__ void load32(const __nv_bfloat16* p, float (&x)[32]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 v = __ldg(reinterpret_cast<const uint4*>(p) + i);
      const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        x[8 * i + 2 * j] = __uint_as_float(w[j] << 16);
        x[8 * i + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
      }
    }
  }
};

// 32 consecutive elements [32 * i, 32 * i + 32) of row `r` of the staged tile (16-bit types): the tile is
// two column halves of [128 rows][128 B], each with the 128-byte swizzle the TMA applied
template <typename T>
__device__ __forceinline__ void load32_tile(const unsigned char* xt, int r, int i, float (&x)[32]) {
#pragma unroll
  for (int cc = 0; cc < 4; ++cc) {
    const int chunk = 4 * i + cc;  // 16-byte chunk of the row (8 elements)
    const uint4 v = *reinterpret_cast<const uint4*>(xt + (chunk >> 3) * kBlockBytes + swz(r, chunk & 7));
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if constexpr (std::is_same<T, __nv_bfloat16>::value) {
        x[8 * cc + 2 * j] = __uint_as_float(w[j] << 16);
        x[8 * cc + 2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
      } else {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
        x[8 * cc + 2 * j] = f.x;
        x[8 * cc + 2 * j + 1] = f.y;
      }
    }
  }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}

// XT: the rows of a source are contiguous 16-bit vectors; the next tile's rows are fetched into
// shared memory by TMA while the current tile is in the tensor core and the epilogue.  Tiles then
// never mix the two sources (the last tile of K may be partly empty).
template <typename T, bool XT>
__global__ void __launch_bounds__(kThreads, 1)
compress_tc_kernel(const CompressArgs a, const __grid_constant__ CUtensorMap tm_x0,
                   const __grid_constant__ CUtensorMap tm_x1) {
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t s_bar[3];  // [0]: first K-step's MMAs done, [1]: tile's MMAs done, [2]: input tile landed
  __shared__ uint32_t s_tmem;
  __shared__ int s_dead;
  __shared__ float s_bounds[2][16];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int row_in_tile = 32 * (warp & 3) + lane;  // = the TMEM lane this thread can read
  const int half = warp >> 2;                      // which 64 columns / which K-block of a K-step
  const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  unsigned char* sm = smem_raw + (base - smem_addr(smem_raw));
  const uint32_t bar0 = smem_addr(&s_bar[0]), bar1 = smem_addr(&s_bar[1]);

  if (tid < 32) {
    const int src = tid >> 4, i = tid & 15;
    s_bounds[src][i] = (src < a.n_sources && i < a.n_bounds[src]) ? a.bounds[src][i] : CUDART_INF_F;
  }
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar0) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar1) : "memory");
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(&s_bar[2])) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_dead = 0;
  }
  if (warp == 0) {  // one warp allocates the accumulator's tensor-memory columns
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&s_tmem)),
                 "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // ---- Pi as the B operand: B[n = j][k = d] = Pi[j][d], hi and lo, K-major swizzled -------------
  // rot_even[k * 64 + p] = Pi[2p][k], rot_odd[k * 64 + p] = Pi[2p + 1][k]
  for (int i = tid; i < kD * kD; i += kThreads) {
    const int k = i >> 7, j = i & 127;
    const float v = __ldg((j & 1 ? a.rot_odd : a.rot_even) + k * (kD / 2) + (j >> 1));
    float hi, lo;
    split_tf32(v, hi, lo);
    const uint32_t off = (uint32_t)(k >> 5) * kBlockBytes + swz(j, (k & 31) >> 2) + (k & 3) * 4;
    *reinterpret_cast<float*>(sm + kOffBhi + off) = hi;
    *reinterpret_cast<float*>(sm + kOffBlo + off) = lo;
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_d = s_tmem;

  const int64_t rows_per_src = a.n_tokens * a.num_heads;
  const int64_t total_rows = rows_per_src * a.n_sources;
  const int64_t tiles_per_src = (rows_per_src + kRows - 1) / kRows;
  const int64_t n_tiles = XT ? tiles_per_src * a.n_sources : (total_rows + kRows - 1) / kRows;
  const RowLayout lay = row_layout(a.num_heads, kD);
  const uint32_t bar_x = smem_addr(&s_bar[2]);
  const unsigned char* xt = sm + kOffX;
  uint32_t phase = 0;
  // XT: one thread fetches the 128 rows of tile `t` (two boxes of 64 columns); rows past the end of
  // the source are zero-filled by the copy
  auto fetch_tile = [&](int64_t t) {
    const int s_ = (int)(t / tiles_per_src);
    const int y = (int)((t - (int64_t)s_ * tiles_per_src) * kRows);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_x), "r"(kXBytes) : "memory");
    tma_load_2d(base + kOffX, s_ ? &tm_x1 : &tm_x0, 0, y, bar_x);
    tma_load_2d(base + kOffX + kBlockBytes, s_ ? &tm_x1 : &tm_x0, 64, y, bar_x);
  };
  if (XT && (int64_t)blockIdx.x < n_tiles && warp == 0 && elect_one_sync()) fetch_tile(blockIdx.x);

  for (int64_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x) {
    int64_t row;
    bool live;
    int src = 0, h = 0;
    int64_t tok = 0;
    const T* xp = nullptr;
    if (XT) {
      src = (int)(tile / tiles_per_src);
      const int64_t in_src = (tile - (int64_t)src * tiles_per_src) * kRows + row_in_tile;
      live = in_src < rows_per_src;
      row = (int64_t)src * rows_per_src + in_src;
    } else {
      row = tile * kRows + row_in_tile;
      live = row < total_rows;
      if (live) src = row >= rows_per_src ? 1 : 0;
    }
    if (live) {
      const unsigned rem = (unsigned)(row - (src ? rows_per_src : 0));
      const unsigned t = rem / (unsigned)a.num_heads;
      tok = t;
      h = (int)(rem - t * (unsigned)a.num_heads);
      xp = reinterpret_cast<const T*>(a.x[src]) + tok * a.token_stride[src] + (int64_t)h * a.head_stride[src];
    }
    // ---- norm, in the summation order of the FMA kernels: p[l] over k = l, l+32, l+64, l+96,
    //      then the butterfly tree 16, 8, 4, 2, 1 -------------------------------------------------
    bool ok = true;
    if (XT) ok = bar_wait_bounded(bar_x, phase);  // the tile's rows have landed
    float nrm = 0.f;
    if (live) {
      float p[32];
#pragma unroll
      for (int l = 0; l < 32; ++l) p[l] = 0.f;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        float x[32];
        if constexpr (XT) load32_tile<T>(xt, row_in_tile, i, x);
        else RowLoader<T>::load32(xp + 32 * i, x);
#pragma unroll
        for (int l = 0; l < 32; ++l) p[l] = fmaf(x[l], x[l], p[l]);
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1)
#pragma unroll
        for (int l = 0; l < o; ++l) p[l] = p[l] + p[l + o];
      nrm = sqrtf(p[0]);
    }
    // one IEEE division per row; x * (1 / den) is within an ulp of x / den, far below the TF32 split error
    const float inv_den = 1.f / (nrm + 1e-10f);

    // ---- two K-steps of 64: this thread fills K-block (2 * step + half) of A into buffer `half` ----
#pragma unroll 1
    for (int step = 0; step < 2; ++step) {
      const int kb = 2 * step + half;
      float x[32];
      if (live) {
        if constexpr (XT) load32_tile<T>(xt, row_in_tile, kb, x);
        else RowLoader<T>::load32(xp + 32 * kb, x);
      } else {
#pragma unroll
        for (int l = 0; l < 32; ++l) x[l] = 0.f;
      }
      if (step == 1) ok = bar_wait_bounded(bar0, phase) && ok;  // the first K-step's MMAs have read the buffers
      unsigned char* a_hi = sm + kOffA + half * (2 * kBlockBytes);
      unsigned char* a_lo = a_hi + kBlockBytes;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        float hi[4], lo[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) split_tf32(x[4 * c + e] * inv_den, hi[e], lo[e]);
        const uint32_t off = swz(row_in_tile, c);
        *reinterpret_cast<float4*>(a_hi + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
        *reinterpret_cast<float4*>(a_lo + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
      }
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // stores -> visible to the tensor core
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      if (!ok) s_dead = 1;
      __syncthreads();
      if (s_dead) break;
      if (warp == 0 && elect_one_sync()) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
        for (int b = 0; b < 2; ++b) {  // the two K-blocks of this step: buffers 0 and 1
          const uint32_t ahi = base + kOffA + b * (2 * kBlockBytes), alo = ahi + kBlockBytes;
          const uint32_t bhi = base + kOffBhi + (2 * step + b) * kBlockBytes;
          const uint32_t blo = base + kOffBlo + (2 * step + b) * kBlockBytes;
#pragma unroll
          for (int s = 0; s < 4; ++s) {  // four MMA K-slices of 8 columns (32 bytes) per K-block
            const uint32_t ko = 32u * s;
            mma_tf32(tmem_d, make_desc(alo + ko), make_desc(bhi + ko), (step | b | s) ? 1u : 0u);
            mma_tf32(tmem_d, make_desc(ahi + ko), make_desc(blo + ko), 1u);
            mma_tf32(tmem_d, make_desc(ahi + ko), make_desc(bhi + ko), 1u);
          }
        }
        mma_commit(step == 0 ? bar0 : bar1);
        // every thread has read its row for the last time: fetch the rows of this CTA's next tile
        if (XT && step == 1 && tile + gridDim.x < n_tiles) fetch_tile(tile + gridDim.x);
      }
    }
    if (s_dead) break;
    // ---- epilogue: this thread's 64 columns of its row ------------------------------------------
    ok = __all_sync(0xffffffffu, bar_wait_bounded(bar1, phase));  // warp-uniform: the loads below are .aligned
    if (!ok) s_dead = 1;  // (every thread that times out writes the same value)
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    phase ^= 1u;
    uint32_t packed[8];  // this thread's 64 indices = 32 bytes
    if (ok) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        uint32_t v[32];
        const uint32_t taddr = tmem_d + ((uint32_t)(32 * (warp & 3)) << 16) + (uint32_t)(64 * half + 32 * q);
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
            "%14, %15, %16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
              "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
              "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
              "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
            : "r"(taddr)
            : "memory");
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        const float* b = s_bounds[src];
#pragma unroll
        for (int w = 0; w < 4; ++w) {  // 8 coordinates -> 4 bytes -> one word
          uint32_t word = 0;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int ie = bucketize_sorted16(__uint_as_float(v[8 * w + 2 * e]), b);
            const int io = bucketize_sorted16(__uint_as_float(v[8 * w + 2 * e + 1]), b);
            word |= (uint32_t)((ie << 4) | io) << (8 * e);
          }
          packed[4 * q + w] = word;
        }
      }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");  // loads done before the next tile's MMAs
    if (ok && live) {
      uint8_t* dst_idx = nullptr;
      float* dst_norm = nullptr;
      if (a.cache != nullptr) {
        const int64_t slot = tok < a.n_slots ? a.slot_mapping[tok] : -1;
        if (slot >= a.num_cache_slots) {
          if (half == 0 && a.err_flag) atomicOr(a.err_flag, TQ4_DEV_BAD_SLOT);
        } else if (slot >= 0) {
          uint8_t* rowp = a.cache + slot * a.cache_token_stride;
          dst_idx = rowp + (src == 0 ? lay.k_idx : lay.v_idx) + h * (kD / 2);
          dst_norm = reinterpret_cast<float*>(rowp + (src == 0 ? lay.k_norm : lay.v_norm) + h * 4);
        }
      } else {
        dst_idx = a.packed_out + row * (kD / 2);
        dst_norm = a.norms_out + row;
      }
      if (dst_idx) {
        uint32_t* d32 = reinterpret_cast<uint32_t*>(dst_idx + 32 * half);  // rows are 4-byte aligned
#pragma unroll
        for (int w = 0; w < 8; ++w) d32[w] = packed[w];
        if (half == 0) *dst_norm = nrm;
      }
    }
  }
  if (s_dead && tid == 0 && a.err_flag) atomicOr(a.err_flag, TQ4_DEV_TIMEOUT);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(kTmemCols) : "memory");
  }
}

}  // namespace

// true if this launch can use the tensor-core kernel
bool compress_tc_eligible(const CompressArgs& a, int head_dim, int dtype) {
  static const bool disabled = getenv("TQ4_NO_TC") != nullptr;
  if (disabled || head_dim != kD) return false;
  const int es = dtype == TQ4_F32 ? 4 : 2;
  for (int s = 0; s < a.n_sources; ++s) {
    if (((uintptr_t)a.x[s] & 15) || (a.token_stride[s] * es) % 16 || (a.head_stride[s] * es) % 16) return false;
  }
  return true;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  }
  return fn;
}
// rows of one source as a 2-D tensor [rows][128] of 16-bit elements; box = 128 rows x 64 columns
static bool make_x_map(CUtensorMap* m, const void* x, int64_t rows) {
  EncodeTiledFn fn = encode_fn();
  if (!fn || rows <= 0) return false;
  const cuuint64_t dims[2] = {(cuuint64_t)kD, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)kD * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)kRows};
  const cuuint32_t estr[2] = {1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(x), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename T, bool XT>
static int launch_tc_t(const CompressArgs& a, const CUtensorMap& m0, const CUtensorMap& m1, cudaStream_t st) {
  const int smem = (int)kSmemBytes + (XT ? (int)kXBytes : 0) + 1024;
  if (!ensure_dynamic_smem<compress_tc_kernel<T, XT>>(smem)) return TQ4_ERR_CUDA;
  const int64_t rows_per_src = a.n_tokens * a.num_heads;
  int64_t blocks = XT ? ((rows_per_src + kRows - 1) / kRows) * a.n_sources
                      : (rows_per_src * a.n_sources + kRows - 1) / kRows;
  if (blocks > sm_count()) blocks = sm_count();
  compress_tc_kernel<T, XT><<<(unsigned)blocks, kThreads, smem, st>>>(a, m0, m1);
  TQ4_CHECK_LAUNCH();
  return TQ4_OK;
}

template <typename T>
static int launch_tc(const CompressArgs& a, cudaStream_t st) {
  CUtensorMap m0, m1;
  memset(&m0, 0, sizeof(m0));
  memset(&m1, 0, sizeof(m1));
  if (sizeof(T) == 2) {
    // staged input tiles need every source to be a dense [rows][128] array
    bool dense = true;
    for (int s = 0; s < a.n_sources; ++s)
      dense = dense && a.head_stride[s] == kD && a.token_stride[s] == (int64_t)a.num_heads * kD;
    const int64_t rows = a.n_tokens * a.num_heads;
    if (dense && make_x_map(&m0, a.x[0], rows) && make_x_map(&m1, a.x[a.n_sources > 1 ? 1 : 0], rows))
      return launch_tc_t<T, true>(a, m0, m1, st);
  }
  return launch_tc_t<T, false>(a, m0, m1, st);
}

int launch_compress_tc(const CompressArgs& a, int dtype, cudaStream_t st) {
  switch (dtype) {
    case TQ4_F32: return launch_tc<float>(a, st);
    case TQ4_F16: return launch_tc<__half>(a, st);
    case TQ4_BF16: return launch_tc<__nv_bfloat16>(a, st);
  }
  return TQ4_ERR_UNSUPPORTED;
}

}  // namespace tq4
