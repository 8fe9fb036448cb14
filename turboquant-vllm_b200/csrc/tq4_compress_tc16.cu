// TQ4 compress for prefill-sized 16-bit inputs at head_dim 128, pipelined on the 5th-generation
// tensor cores.  The rotation of a tile of 128 vectors is a 128 x 128 x 128 GEMM
//     Y_raw = X * Pi^T        (tcgen05.mma kind::f16, fp32 accumulator in tensor memory)
// on the RAW input rows: a 16-bit input is exact as an MMA operand, so the A operand needs no
// CUDA-core preparation at all and arrives in shared memory by TMA in the swizzled layout the MMA
// reads.  Pi is the B operand, resident in shared memory as a sum of 16-bit terms (bf16 inputs:
// three bf16 terms = 24 bits; fp16 inputs: 2^8 * Pi as fp16 hi + lo = 22 bits), one MMA per term.
// The normalisation commutes with the product: y = Y_raw / (norm + 1e-10) is applied to the fp32
// accumulator in the epilogue.  A rotated coordinate therefore differs from the fp32 FMA kernels by
// ~1e-7 absolute, which moves an index only when the coordinate sits that close to a bucket
// boundary (bound 1e-4 of the indices).  Norms are summed in exactly the order of the FMA kernels
// (lane-strided FMAs, butterfly tree), so they are bit-identical to them.
//
// One persistent CTA per SM, warp-specialised, four input stages and four accumulators in flight:
//   warp 0      TMA producer: the 128 rows of a tile as two 64-column boxes (128-byte swizzle)
//   warp 1      MMA issuer: 8 k-steps x terms of tcgen05.mma 128x128x16, then tcgen05.commit onto
//               the stage's "empty" barrier and the accumulator's "full" barrier
//   warps 2-17  four epilogue groups of four warps; tile i of the CTA belongs to group i % 4 and uses
//               input stage i % 4 and accumulator i % 4, so every barrier is waited on by one group
//               in tile order (a stage shared between groups could show a fast group an older
//               phase).  The epilogue is CUDA-core work; four warps per scheduler hide its latencies:
//               thread = row.  Sum of squares from the staged tile -> release the stage -> wait for
//               the accumulator -> four times: tcgen05.ld of 32 columns, scale, bucketize (binary
//               search over boundaries held in registers), nibble-pack, one 16-byte store into the
//               packed output or the paged cache row.
// Every mbarrier wait is bounded; a wait that gives up marks the CTA dead, all roles drain and the
// kernel reports TQ4_DEV_TIMEOUT.  Tensor memory is released on every path.
#include <cuda.h>
#include <math_constants.h>

#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "tq4_common.cuh"

namespace tq4 {
#ifdef TQ4_TRACE
// Tuning builds only (-DTQ4_TRACE): SM clock at points of the tile pipeline of CTA 0 (producer warp,
// MMA warp, first warp of epilogue groups 0 and 1), read back with tq4_compress_trace_read.
__device__ long long g_ctrace[4][32][8];
#define CT_STAMP(role, i, e)                                                                   \
  do {                                                                                         \
    if (blockIdx.x == 0 && (threadIdx.x & 31) == 0 && (i) < 32) g_ctrace[role][i][e] = clock64(); \
  } while (0)
#else
#define CT_STAMP(role, i, e) do {} while (0)
#endif

namespace {

constexpr int kD = 128;
constexpr int kRows = 128;                       // vectors per tile (MMA M, TMEM lanes)
constexpr int kStages = 4;                       // input stages = epilogue groups = accumulators
constexpr int kAccs = kStages;                   // tile i of a CTA uses stage, accumulator and group i % 4
constexpr int kThreads = 64 + kAccs * 128;       // producer, issuer, kAccs x 4 epilogue warps
constexpr uint32_t kBlockBytes = kRows * 128;    // one K-block (64 16-bit columns) of an operand: 16 KB
constexpr uint32_t kTileBytes = 2 * kBlockBytes; // a tile = two K-blocks
constexpr int kMaxTerms = 3;
constexpr uint32_t kOffB = 0;                                  // terms x 2 K-blocks of Pi
constexpr uint32_t kOffA = kMaxTerms * kTileBytes;             // stages x 2 K-blocks of X
constexpr uint32_t kSmemBytes = kOffA + kStages * kTileBytes;  // 96 KB of Pi terms + 128 KB of input stages
constexpr uint32_t kTmemCols = kAccs * 128;                    // one accumulator of 128 fp32 columns per group

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
// byte offset of (row, 16-byte chunk c of the row's 128 bytes) inside a K-block (128-byte swizzle)
__device__ __forceinline__ uint32_t swz(int row, int c) { return (uint32_t)(row * 128 + ((c ^ (row & 7)) << 4)); }
// K-major operand, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// instruction descriptor: D = F32, A and B of 16-bit format `fmt` (0 = fp16, 1 = bf16), K-major, N = M = 128
__host__ __device__ constexpr uint32_t instr_desc(uint32_t fmt) {
  return (1u << 4) | (fmt << 7) | (fmt << 10) | ((128u >> 3) << 17) | ((128u >> 4) << 24);
}
__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "l"(da), "l"(db), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
      : "memory");
}
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void bar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait that also gives up as soon as another role has marked the CTA dead.
__device__ __forceinline__ bool bar_wait_bounded(uint32_t bar, uint32_t parity, const volatile int* dead) {
  for (int it = 0; it < (1 << 22); ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done) : "r"(bar), "r"(parity) : "memory");
    if (done) return true;
    if ((it & 1023) == 1023 && *dead) return false;
  }
  return false;
}
__device__ __forceinline__ bool elect_one_sync() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
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
}

template <typename T>
struct Fmt;  // how Pi is split into 16-bit terms for inputs of type T
template <>
struct Fmt<__half> {
  static constexpr int kTerms = 2;
  static constexpr uint32_t kCode = 0;
  static constexpr float kScale = 256.f;  // keeps the lo term of small entries a normal fp16 number
  static __device__ __forceinline__ uint16_t term(float& rest) {
    const __half h = __float2half_rn(rest);
    rest -= __half2float(h);
    return __half_as_ushort(h);
  }
};
template <>
struct Fmt<__nv_bfloat16> {
  static constexpr int kTerms = 3;
  static constexpr uint32_t kCode = 1;
  static constexpr float kScale = 1.f;
  static __device__ __forceinline__ uint16_t term(float& rest) {
    const __nv_bfloat16 h = __float2bfloat16_rn(rest);
    rest -= __bfloat162float(h);
    return __bfloat16_as_ushort(h);
  }
};

// eight 16-bit elements (one 16-byte chunk) -> fp32
template <typename T>
__device__ __forceinline__ void chunk_to_float(const uint4& v, float (&x)[8]) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      x[2 * j] = __uint_as_float(w[j] << 16);
      x[2 * j + 1] = __uint_as_float(w[j] & 0xFFFF0000u);
    } else {
      const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
      x[2 * j] = f.x;
      x[2 * j + 1] = f.y;
    }
  }
}

// idx = #{b : b < y} over 15 ascending boundaries (padded with +inf) held in REGISTERS: a four-level
// binary search whose next boundary is picked with selects, so nothing in it touches memory (the
// shared-memory version is a chain of four dependent loads per coordinate, which two epilogue
// warps per scheduler cannot hide).  NaN compares false at every level -> 0.
__device__ __forceinline__ int bucketize_reg(float y, const float (&b)[15]) {
  const bool c1 = y > b[7];
  const bool c2 = y > (c1 ? b[11] : b[3]);
  const float t3 = c2 ? (c1 ? b[13] : b[5]) : (c1 ? b[9] : b[1]);
  const bool c3 = y > t3;
  const float lo4 = c2 ? (c1 ? b[12] : b[4]) : (c1 ? b[8] : b[0]);
  const float hi4 = c2 ? (c1 ? b[14] : b[6]) : (c1 ? b[10] : b[2]);
  const bool c4 = y > (c3 ? hi4 : lo4);
  return (c1 ? 8 : 0) + (c2 ? 4 : 0) + (c3 ? 2 : 0) + (c4 ? 1 : 0);
}

// The same search with the two lower levels as table lookups through the warp shuffle: lane l holds
// boundary l & 15 (`bval`; entry 15 = +inf), and __shfl_sync with a per-thread source lane is a
// 16-entry lookup in one instruction.  Levels 1 and 2 compare against registers (b[7]; b[3] or b[11]);
// 11 instructions per coordinate instead of 22, same comparisons, same result.  The shuffle unit
// cannot take every coordinate (all of them through it: no faster than the register search), so the
// epilogue sends every second one.
__device__ __forceinline__ int bucketize_shfl(float y, float b7, float b3, float b11, float bval) {
  const bool c1 = y > b7;
  int idx = c1 ? 8 : 0;
  idx += (y > (c1 ? b11 : b3)) ? 4 : 0;
  idx += (y > __shfl_sync(0xffffffffu, bval, idx + 1)) ? 2 : 0;
  idx += (y > __shfl_sync(0xffffffffu, bval, idx)) ? 1 : 0;
  return idx;
}

struct Bars {
  uint64_t full[kStages];    // TMA -> consumers: the stage's tile has landed
  uint64_t empty[kStages];   // consumers -> TMA: MMAs (1 commit) and the norm readers (4 warps) are done with it
  uint64_t tfull[kAccs];     // MMA -> epilogue: the accumulator holds the tile's product
  uint64_t tempty[kAccs];    // epilogue (4 warps) -> MMA: the accumulator has been read
  uint64_t pi;               // the raw rotation matrix has landed in the staging area
};

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
compress_tc16_kernel(const CompressArgs a, const __grid_constant__ CUtensorMap tm_x0,
                     const __grid_constant__ CUtensorMap tm_x1) {
  using F = Fmt<T>;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) Bars s_bars;
  __shared__ uint32_t s_tmem;
  __shared__ int s_dead;
  __shared__ float s_bounds[2][16];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (warp == 0) CT_STAMP(0, 31, 6);  // kernel entry
  const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;  // swizzle atoms need 1024-byte alignment
  unsigned char* sm = smem_raw + (base - smem_addr(smem_raw));
  volatile int* dead = &s_dead;

  if (tid < 32) {
    const int src = tid >> 4, i = tid & 15;
    s_bounds[src][i] = (src < a.n_sources && i < a.n_bounds[src]) ? a.bounds[src][i] : CUDART_INF_F;
  }
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      bar_init(smem_addr(&s_bars.full[s]), 1);
      bar_init(smem_addr(&s_bars.empty[s]), 1 + 4);
    }
    for (int c = 0; c < kAccs; ++c) {
      bar_init(smem_addr(&s_bars.tfull[c]), 1);
      bar_init(smem_addr(&s_bars.tempty[c]), 4);
    }
    bar_init(smem_addr(&s_bars.pi), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    s_dead = 0;
    // the caller's Pi^T halves (2 x 32 KB fp32) by two bulk copies into the still unused input stages
    const uint32_t bar = smem_addr(&s_bars.pi);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(2u * kD * (kD / 2) * 4u) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(base + kOffA), "l"(a.rot_even), "r"((uint32_t)(kD * (kD / 2) * 4)), "r"(bar) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(base + kOffA + (uint32_t)(kD * (kD / 2) * 4)), "l"(a.rot_odd), "r"((uint32_t)(kD * (kD / 2) * 4)), "r"(bar) : "memory");
  }
  if (warp == 1) {  // the issuing warp owns the tensor-memory allocation
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&s_tmem)),
                 "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // ---- Pi as the B operand: B[n = j][k = d] = Pi[j][d] in 16-bit terms, K-major, swizzled ---------
  // rot_even[k * 64 + p] = Pi[2p][k], rot_odd[k * 64 + p] = Pi[2p + 1][k], read from the staging area
  __syncthreads();  // the barrier is initialised, the copies are issued, the boundaries are in shared memory
  const bool pi_ok = bar_wait_bounded(smem_addr(&s_bars.pi), 0u, &s_dead);
  const float* raw = reinterpret_cast<const float*>(sm + kOffA);
  for (int i = tid; i < kD * (kD / 8); i += kThreads) {
    const int j = i & 127, k8 = i >> 7;  // row j, k = 8 * k8 .. + 7
    const float* src = raw + (j & 1) * (kD * (kD / 2)) + (j >> 1);
    uint16_t t[kMaxTerms][8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      float rest = src[(8 * k8 + e) * (kD / 2)] * F::kScale;
#pragma unroll
      for (int m = 0; m < F::kTerms; ++m) t[m][e] = F::term(rest);
    }
    const uint32_t off = (uint32_t)(k8 >> 3) * kBlockBytes + swz(j, k8 & 7);
#pragma unroll
    for (int m = 0; m < F::kTerms; ++m) {
      uint4 v;
      v.x = t[m][0] | ((uint32_t)t[m][1] << 16);
      v.y = t[m][2] | ((uint32_t)t[m][3] << 16);
      v.z = t[m][4] | ((uint32_t)t[m][5] << 16);
      v.w = t[m][6] | ((uint32_t)t[m][7] << 16);
      *reinterpret_cast<uint4*>(sm + kOffB + m * kTileBytes + off) = v;
    }
  }
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = s_tmem;
  if (warp == 0) CT_STAMP(0, 31, 7);  // set-up done (Pi converted, tensor memory allocated)

  const int64_t rows_per_src = a.n_tokens * a.num_heads;
  const int64_t tiles_per_src = (rows_per_src + kRows - 1) / kRows;
  const int64_t n_tiles = tiles_per_src * a.n_sources;
  const int64_t my_tiles = (int64_t)blockIdx.x < n_tiles ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  bool ok = pi_ok;

  if (warp == 0) {
    // ================= TMA producer =================
    for (int64_t i = 0; i < my_tiles && ok; ++i) {
      const int st = (int)(i % kStages);
      const uint32_t par = (uint32_t)((i / kStages) & 1);
      // (passes at once the first time round; warp-uniform so that the election below is well formed)
      ok = __all_sync(0xffffffffu, bar_wait_bounded(smem_addr(&s_bars.empty[st]), par ^ 1u, dead));
      if (!ok) break;
      CT_STAMP(0, i, 0);
      if (elect_one_sync()) {
        const int64_t tile = blockIdx.x + i * gridDim.x;
        const int s_ = (int)(tile / tiles_per_src);
        const int y = (int)((tile - (int64_t)s_ * tiles_per_src) * kRows);
        const uint32_t bar = smem_addr(&s_bars.full[st]);
        const uint32_t dst = base + kOffA + st * kTileBytes;
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(kTileBytes) : "memory");
        tma_load_2d(dst, s_ ? &tm_x1 : &tm_x0, 0, y, bar);            // rows past the end are zero-filled
        tma_load_2d(dst + kBlockBytes, s_ ? &tm_x1 : &tm_x0, 64, y, bar);
      }
      __syncwarp();
    }
  } else if (warp == 1) {
    // ================= MMA issuer =================
    constexpr uint32_t idesc = instr_desc(F::kCode);
    for (int64_t i = 0; i < my_tiles && ok; ++i) {
      const int st = (int)(i % kStages), acc = (int)(i % kAccs);
      ok = __all_sync(0xffffffffu,
                      bar_wait_bounded(smem_addr(&s_bars.full[st]), (uint32_t)((i / kStages) & 1), dead) &&
                          bar_wait_bounded(smem_addr(&s_bars.tempty[acc]), (uint32_t)((i / kAccs) & 1) ^ 1u, dead));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      CT_STAMP(1, i, 0);
      if (elect_one_sync()) {
        const uint32_t tmem_d = tmem_base + (uint32_t)acc * kD;
        const uint32_t a0 = base + kOffA + st * kTileBytes;
#pragma unroll
        for (int m = F::kTerms - 1; m >= 0; --m) {  // smallest term first
          const uint32_t b0 = base + kOffB + m * kTileBytes;
#pragma unroll
          for (int kb = 0; kb < 2; ++kb)
#pragma unroll
            for (int s = 0; s < 4; ++s) {  // four k-steps of 16 columns (32 bytes) per K-block
              const uint32_t ko = kb * kBlockBytes + 32u * s;
              mma_f16(tmem_d, make_desc(a0 + ko), make_desc(b0 + ko), idesc, (m != F::kTerms - 1 || kb || s) ? 1u : 0u);
            }
        }
        mma_commit(smem_addr(&s_bars.empty[st]));   // the tensor core has read the stage
        mma_commit(smem_addr(&s_bars.tfull[acc]));  // the accumulator is complete
      }
      __syncwarp();
      CT_STAMP(1, i, 1);
    }
  } else {
    // ================= epilogue groups =================
    const int grp = (warp - 2) >> 2;              // tiles i with i % kAccs == grp, accumulator grp
    const int quarter = warp & 3;                 // the 32 TMEM lanes this warp may read
    const int row_in_tile = 32 * quarter + lane;
    const RowLayout lay = row_layout(a.num_heads, kD);
    for (int64_t i = grp; i < my_tiles && ok; i += kAccs) {
      const int st = (int)(i % kStages), acc = grp;
      const int64_t tile = blockIdx.x + i * gridDim.x;
      const int src = (int)(tile / tiles_per_src);
      const int64_t in_src = (tile - (int64_t)src * tiles_per_src) * kRows + row_in_tile;
      const bool live = in_src < rows_per_src;
      ok = __all_sync(0xffffffffu, bar_wait_bounded(smem_addr(&s_bars.full[st]), (uint32_t)((i / kStages) & 1), dead));
      if (!ok) break;
      if (quarter == 0 && grp < 2) CT_STAMP(2 + grp, i, 0);
      // ---- norm, in the summation order of the FMA kernels: p[l] over k = l, l+32, l+64, l+96,
      //      then the butterfly tree 16, 8, 4, 2, 1 --------------------------------------------------
      float nrm = 0.f;
      {
        const unsigned char* xt = sm + kOffA + st * kTileBytes;
        float p[32];
#pragma unroll
        for (int l = 0; l < 32; ++l) p[l] = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {  // elements [32 q, 32 q + 32) of the row
#pragma unroll
          for (int cc = 0; cc < 4; ++cc) {
            const int chunk = 4 * q + cc;
            const uint4 v = *reinterpret_cast<const uint4*>(xt + (chunk >> 3) * kBlockBytes + swz(row_in_tile, chunk & 7));
            float x[8];
            chunk_to_float<T>(v, x);
#pragma unroll
            for (int e = 0; e < 8; ++e) p[8 * cc + e] = fmaf(x[e], x[e], p[8 * cc + e]);
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
          for (int l = 0; l < o; ++l) p[l] = p[l] + p[l + o];
        nrm = sqrtf(p[0]);
      }
      __syncwarp();
      if (quarter == 0 && grp < 2) CT_STAMP(2 + grp, i, 1);
      if (lane == 0) bar_arrive(smem_addr(&s_bars.empty[st]));  // this warp is done with the staged rows
      // one IEEE division per row; Y_raw * (1 / den) is within an ulp of Y_raw / den
      const float scale = (1.f / (nrm + 1e-10f)) * (1.f / F::kScale);
      // where this row goes (resolved before the accumulator is read: the loads overlap the wait)
      uint8_t* dst_idx = nullptr;
      float* dst_norm = nullptr;
      if (live) {
        const unsigned rem = (unsigned)in_src;
        const unsigned tok = rem / (unsigned)a.num_heads;
        const int h = (int)(rem - tok * (unsigned)a.num_heads);
        if (a.cache != nullptr) {
          const int64_t slot = (int64_t)tok < a.n_slots ? a.slot_mapping[tok] : -1;
          if (slot >= a.num_cache_slots) {
            if (a.err_flag) atomicOr(a.err_flag, TQ4_DEV_BAD_SLOT);
          } else if (slot >= 0) {
            uint8_t* rowp = a.cache + slot * a.cache_token_stride;
            dst_idx = rowp + (src == 0 ? lay.k_idx : lay.v_idx) + h * (kD / 2);
            dst_norm = reinterpret_cast<float*>(rowp + (src == 0 ? lay.k_norm : lay.v_norm) + h * 4);
          }
        } else {
          const int64_t row = (int64_t)src * rows_per_src + in_src;
          dst_idx = a.packed_out + row * (kD / 2);
          dst_norm = a.norms_out + row;
        }
      }
      float b[15];
#pragma unroll
      for (int bi = 0; bi < 15; ++bi) b[bi] = s_bounds[src][bi];
      const float bval = s_bounds[src][lane & 15];  // (entry 15 is +inf)
      const bool wide = dst_idx != nullptr && ((uintptr_t)dst_idx & 15) == 0;  // else rows are 4-byte aligned

      ok = __all_sync(0xffffffffu, bar_wait_bounded(smem_addr(&s_bars.tfull[acc]), (uint32_t)((i / kAccs) & 1), dead));
      if (!ok) break;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (quarter == 0 && grp < 2) CT_STAMP(2 + grp, i, 2);
      // four chunks of 32 coordinates -> 16 bytes each; the loop stays rolled so that its body (32
      // register searches) fits the instruction cache
#pragma unroll 1
      for (int q = 0; q < 4; ++q) {
        uint32_t v[32];
        tmem_ld32(tmem_base + ((uint32_t)(32 * quarter) << 16) + (uint32_t)(acc * kD + 32 * q), v);
        uint32_t word[4];
#pragma unroll
        for (int w = 0; w < 4; ++w) {  // 8 coordinates -> 4 bytes -> one word
          word[w] = 0;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int ie = bucketize_reg(__uint_as_float(v[8 * w + 2 * e]) * scale, b);
            const int io = bucketize_shfl(__uint_as_float(v[8 * w + 2 * e + 1]) * scale, b[7], b[3], b[11], bval);
            word[w] |= (uint32_t)((ie << 4) | io) << (8 * e);
          }
        }
        if (wide) {
          reinterpret_cast<uint4*>(dst_idx)[q] = make_uint4(word[0], word[1], word[2], word[3]);
        } else if (dst_idx) {
#pragma unroll
          for (int w = 0; w < 4; ++w) reinterpret_cast<uint32_t*>(dst_idx)[4 * q + w] = word[w];
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) bar_arrive(smem_addr(&s_bars.tempty[acc]));  // the accumulator may be overwritten
      if (dst_norm) *dst_norm = nrm;
      if (quarter == 0 && grp < 2) CT_STAMP(2 + grp, i, 3);
    }
  }
  if (!ok) {
    s_dead = 1;
    if (lane == 0 && a.err_flag) atomicOr(a.err_flag, TQ4_DEV_TIMEOUT);
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 1) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn encode_fn() {
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
bool make_x_map(CUtensorMap* m, const void* x, int64_t rows) {
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

template <typename T>
int launch_t(const CompressArgs& a, cudaStream_t st) {
  CUtensorMap m0, m1;
  memset(&m0, 0, sizeof(m0));
  memset(&m1, 0, sizeof(m1));
  const int64_t rows = a.n_tokens * a.num_heads;
  if (!make_x_map(&m0, a.x[0], rows) || !make_x_map(&m1, a.x[a.n_sources > 1 ? 1 : 0], rows))
    return TQ4_ERR_CUDA;
  const int smem = (int)kSmemBytes + 1024;
  if (!ensure_dynamic_smem<compress_tc16_kernel<T>>(smem)) return TQ4_ERR_CUDA;
  int64_t blocks = ((rows + kRows - 1) / kRows) * a.n_sources;
  if (blocks > sm_count()) blocks = sm_count();
  compress_tc16_kernel<T><<<(unsigned)blocks, kThreads, smem, st>>>(a, m0, m1);
  TQ4_CHECK_LAUNCH();
  return TQ4_OK;
}

}  // namespace

// 16-bit inputs whose rows are dense [tokens * heads][128] arrays (the layout vLLM hands to the cache
// write): the pipelined kernel.  Everything else stays on the kernels in tq4_compress_tc.cu / tq4_compress.cu.
bool compress_tc16_eligible(const CompressArgs& a, int head_dim, int dtype) {
  static const bool disabled = getenv("TQ4_NO_TC") != nullptr || getenv("TQ4_NO_TC16") != nullptr;
  if (disabled || head_dim != kD || (dtype != TQ4_F16 && dtype != TQ4_BF16)) return false;
  if (a.n_tokens * a.num_heads >= (1ll << 31) || encode_fn() == nullptr) return false;
  for (int s = 0; s < a.n_sources; ++s) {
    if (((uintptr_t)a.x[s] & 15) || a.head_stride[s] != kD || a.token_stride[s] != (int64_t)a.num_heads * kD)
      return false;
  }
  if (((uintptr_t)a.rot_even | (uintptr_t)a.rot_odd) & 15) return false;  // bulk copies of the rotation halves
  return true;
}

int launch_compress_tc16(const CompressArgs& a, int dtype, cudaStream_t st) {
  return dtype == TQ4_F16 ? launch_t<__half>(a, st) : launch_t<__nv_bfloat16>(a, st);
}

}  // namespace tq4

#ifdef TQ4_TRACE
extern "C" int tq4_compress_trace_read(long long* out) {
  return cudaMemcpyFromSymbol(out, tq4::g_ctrace, sizeof(long long) * 4 * 32 * 8) == cudaSuccess ? 0 : 1;
}
#endif
