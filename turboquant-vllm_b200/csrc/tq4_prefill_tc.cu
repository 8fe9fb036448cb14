// Chunked-prefill attention over the packed TQ4 cache on the 5th-generation tensor cores
// (head_dim 128).  A CTA owns a block of 128 / G query rows of one sequence and one KV head: the
// M = 128 rows of the MMAs are the (query row, query head of the GQA group) pairs, so a key/value
// tile is dequantised ONCE per CTA and serves all of them (the streaming kernel dequantises it per
// query row).  Everything happens in rotated space on the queries the prologue kernel rotated.
//
// Per 64-token tile:
//   TMA boxes (K+V index rows and norm columns of 4 pages)                      -> shared memory
//   dequantise through a 256-entry byte -> half2 table: K~ [64 tok][128 d] and V~ as fp16,
//     stored in the swizzled layouts the MMA descriptors expect                  CUDA cores
//   S = Qhi K~^T + Qlo K~^T   (tcgen05.mma kind::f16, 128 x 64 x 16, fp32 in TMEM, two S buffers)
//   tcgen05.ld S, x knorm, mask, lazy online softmax, P = p * vnorm as fp16 hi + lo   CUDA cores
//   O += Plo V~ + Phi V~      (tcgen05.mma 128 x 128 x 16, V~ as an MN-major B operand)
// The A operands of both products live in TENSOR MEMORY, not in shared memory: the block's queries
// are written there once (tcgen05.st, two fp16 per 32-bit column), the probabilities once per tile by
// the threads that computed them.  The loop is bound by shared-memory bandwidth (the tensor pipe
// fetches its shared-memory operands again for every instruction, beside the dequantisation's own
// loads and stores): with Q and P in shared memory the MMAs alone read 224 KB per tile, now 96 KB.
// At the end the normalised rows (still rotated) and their log-sum-exp go to the scratch in the
// layout of one dense partial per row; the merge kernel un-rotates and stores them.
// The first 4 * kTPR warps own the S / O rows, kTPR threads per row (softmax, rescale, epilogue; kTPR = 2:
// with four threads per row the softmax part shortens but the 24 warps slow the dequantisation down
// more); the next eight warps dequantise the following tile into the other K~ / V~ buffer meanwhile
// (keys first, so that the next scores can be issued early; then the values).  One thread of the first
// of them issues the MMAs; one thread of each of the last four issues the TMA copies of one page.
// (A warp for the issuing alone was tried: five warps on one scheduler cut the register budget to 96
// and the loop ran no faster.)  Every wait is bounded.
#include <cuda.h>
#include <math_constants.h>

#include <cstdlib>
#include <cstring>
#include <type_traits>

#include "tq4_attention.cuh"

namespace tq4 {
#ifdef TQ4_TRACE
// Tuning builds only (-DTQ4_TRACE): the SM clock at points of the tile loop, for four warps of one
// CTA, read back with tq4_prefill_trace_read.  Compiled out of the shipped library.
__device__ long long g_ptrace[4][64][16];
#define PF_STAMP(j, e)                                                                              \
  do {                                                                                              \
    if (blockIdx.x == 40 && blockIdx.y == 3 && lane == 0 && (j) < 64 &&                             \
        (warp == 0 || warp == 4 || warp == TQ4_PREFILL_TPR * 4 || warp == TQ4_PREFILL_TPR * 4 + 7))       \
      g_ptrace[warp == 0 ? 0 : warp == 4 ? 1 : warp == TQ4_PREFILL_TPR * 4 ? 2 : 3][j][e] = clock64();  \
  } while (0)
#else
#define PF_STAMP(j, e) do {} while (0)
#endif
namespace {

constexpr int kD = 128;
constexpr int kBN = 64;                 // tokens per tile
#ifndef TQ4_PREFILL_TPR
#define TQ4_PREFILL_TPR 2
#endif
constexpr int kTPR = TQ4_PREFILL_TPR;     // softmax threads per row (2 or 4)
constexpr int kCols = kBN / kTPR;         // score columns per softmax thread
constexpr int kOCols = kD / kTPR;         // output columns per softmax thread
constexpr int kSmx = 128 * kTPR;          // softmax warps 0 .. 4 kTPR - 1
constexpr int kDeq = 256;                 // then eight warps that dequantise
constexpr int kThreads = kSmx + kDeq;
constexpr int kIssueWarp = kSmx / 32;     // one thread of warp 8 also issues the MMAs,
constexpr int kCopyWarp = kThreads / 32 - 1;  // the last four warps issue the TMA copies, one page each
// tensor memory (all 512 columns: one CTA per SM): S (two buffers) [0, 64) and [64, 128), O [128, 256),
// Q hi [256, 320) and lo [320, 384) (128 dims, two per column), P hi [384, 416) and lo [416, 448)
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 128, kColQ = 256, kColQlo = 320, kColP = 384, kColPlo = 416;

// shared-memory map (offsets from a 1024-byte aligned base)
constexpr uint32_t kOffK = 0;                         // 2 buffers x 2 K-blocks x [64 tok][128 B]
constexpr uint32_t kOffV = kOffK + 32768;             // 2 buffers x 2 MN-blocks x [64 tok][128 B]
constexpr uint32_t kOffStage = kOffV + 32768;         // 2 x (4 pages x 2048 B indices + 4 x 512 B norms)
constexpr uint32_t kStageBytes = 4 * 2048 + 4 * 512;
// byte -> half2 tables of K and V, 32 copies of every entry side by side: lane l reads copy l, so a
// warp's 32 lookups always hit 32 different banks (with 16 copies 43 % of the kernel's shared-memory
// wavefronts were conflicts of these lookups)
constexpr int kLutCopies = 32;
constexpr uint32_t kOffLut = kOffStage + 2 * kStageBytes;   // 2 tables x 256 entries x 16 copies x 4 B
constexpr uint32_t kOffNorm = kOffLut + 2 * 256 * kLutCopies * 4;  // 2 buffers x (kn[64], vn[64], lg[64])
constexpr uint32_t kOffXchg = kOffNorm + 2 * 3 * 64 * 4;     // [4][128 rows] floats exchanged by the threads of a row
constexpr uint32_t kSmemBytes = kOffXchg + 4 * 128 * 4;
static_assert(2 * (kSmemBytes + 1024) > 227 * 1024, "one CTA per SM: it allocates the whole tensor memory");

// instruction descriptors (kind::f16, fp16 operands, fp32 accumulator, M = 128)
constexpr uint32_t kDescS = (1u << 4) | ((64u >> 3) << 17) | ((128u >> 4) << 24);                // N = 64, B K-major
constexpr uint32_t kDescO = (1u << 4) | (1u << 16) | ((128u >> 3) << 17) | ((128u >> 4) << 24);  // N = 128, B MN-major

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t swz(int row, int c) { return (uint32_t)(row * 128 + ((c ^ (row & 7)) << 4)); }

// K-major operand, 128-byte swizzle: 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// MN-major operand, 128-byte swizzle: 64-element MN blocks `lbo` bytes apart, 8-row K groups 1024 bytes apart
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr, uint32_t lbo) {
  return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(1024 >> 4) << 32) |
         ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
// D (tensor memory) (+)= A * B with the A operand (128 rows x 16 fp16 = 8 columns) read from tensor memory
__device__ __forceinline__ void mma_f16_ta(uint32_t tmem_d, uint32_t tmem_a, uint64_t db, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
      ::"r"(tmem_d), "r"(tmem_a), "l"(db), "r"(idesc), "r"(acc), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
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
__device__ __forceinline__ bool elect_one_sync() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, int w,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar)
      : "memory");
}
// 32 consecutive fp32 columns of this thread's TMEM lane
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
// 16 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
      "%14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// 8 consecutive 32-bit columns of this thread's TMEM lane (no wait: the caller waits once)
__device__ __forceinline__ void tmem_ld16_nowait(uint32_t taddr, uint32_t (&v)[16]) {  // the caller waits
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, "
      "%14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
// wait for the loads in flight; the registers are named so that no use of them moves above the wait
__device__ __forceinline__ void tmem_ld_wait16(uint32_t (&v)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(v[0]), "+r"(v[1]), "+r"(v[2]), "+r"(v[3]), "+r"(v[4]), "+r"(v[5]), "+r"(v[6]), "+r"(v[7]),
                 "+r"(v[8]), "+r"(v[9]), "+r"(v[10]), "+r"(v[11]), "+r"(v[12]), "+r"(v[13]), "+r"(v[14]), "+r"(v[15])
               :
               : "memory");
}
__device__ __forceinline__ void tmem_st8_nowait(uint32_t taddr, const uint32_t (&v)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, "
      "%15, %16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2_approx(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// G = query heads per KV head (1, 2, 4 or 8); a block holds RB = 128 / G query rows.
// FAST: the queries and the probabilities enter the MMAs as ONE fp16 term each instead of hi + lo
// (half the tensor work and no remainder arithmetic; their rounding, 2^-11 relative, then reaches
// the output: about 1e-3 absolute instead of 1e-5).
template <int G, bool FAST>
__global__ void __launch_bounds__(kThreads, 1)
prefill_tc_kernel(const AttnArgs a, const __grid_constant__ CUtensorMap tm_idx,
                  const __grid_constant__ CUtensorMap tm_norm) {
  constexpr int RB = 128 / G;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ __align__(8) uint64_t s_bar[5];  // [0], [1]: tile stages (TMA), [2], [3]: S buffer ready, [4]: PV done
  __shared__ uint32_t s_tmem;
  __shared__ int s_info[4];                   // sequence, first local row, rows in block, dead flag
  const AttnShape& sh = a.sh;
  const AttnPlan& p = a.plan;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int kvh = blockIdx.y;

  pdl_trigger();
  pdl_wait();  // plan and rotated queries come from the prologue kernel, the cache from the write

  // ---- which (sequence, row block) is this CTA's? ----------------------------------------------
  if (tid == 0) {
    const int lo_all = sh.row_offset, hi_all = sh.row_offset + sh.rows;
    int acc = 0, found = -1, first = 0, nrows = 0;
    for (int s = 0; s < sh.num_seqs && found < 0; ++s) {
      const int q0 = max(a.query_start_loc[s], lo_all), q1 = min(a.query_start_loc[s + 1], hi_all);
      if (q1 <= q0) continue;
      const int nb = (q1 - q0 + RB - 1) / RB;
      if ((int)blockIdx.x < acc + nb) {
        found = s;
        first = q0 + ((int)blockIdx.x - acc) * RB;
        nrows = min(RB, q1 - first);
      }
      acc += nb;
    }
    s_info[0] = found;
    s_info[1] = first - sh.row_offset;
    s_info[2] = nrows;
    s_info[3] = 0;
  }
  __syncthreads();
  const int seq = s_info[0], lr0 = s_info[1], nrows = s_info[2];
  if (seq < 0) return;  // grid is an upper bound on the number of blocks

  const uint32_t base = (smem_addr(smem_raw) + 1023u) & ~1023u;
  unsigned char* sm = smem_raw + (base - smem_addr(smem_raw));
  const uint32_t bar_t0 = smem_addr(&s_bar[0]), bar_s0 = smem_addr(&s_bar[2]), bar_o = smem_addr(&s_bar[4]);
  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < 5; ++i)
      asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar_t0 + 8 * i) : "memory");
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (warp == 0) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&s_tmem)),
                 "r"(kTmemCols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  // byte -> half2 tables: (centroid[hi nibble], centroid[lo nibble]) scaled onto the fp16 grid
  {
    uint32_t* lut = reinterpret_cast<uint32_t*>(sm + kOffLut);
    for (int i = tid; i < 512 * kLutCopies; i += kThreads) {
      const int e = i / kLutCopies, w = e >> 8, b = e & 255;
      const float* cent = w ? a.v_centroids : a.k_centroids;
      const int nc = w ? a.n_v_centroids : a.n_k_centroids;
      const float sc = w ? a.lut_scale_v : a.lut_scale_k;
      const float c_hi = (b >> 4) < nc ? __fmul_rn(sc, cent[b >> 4]) : 0.f;
      const float c_lo = (b & 15) < nc ? __fmul_rn(sc, cent[b & 15]) : 0.f;
      lut[i] = pack_h2(c_hi, c_lo);
    }
  }
  // ---- the block's queries: row m = r * G + g = tensor-memory lane m, scaled by 1 / max|q|, split into
  //      fp16 hi + lo, two dims per 32-bit column.  A warp reaches lanes 32 * (warp % 4) ..., so thread
  //      (warp, lane) stages dims [32 * (warp / 4), + 32) of row 32 * (warp % 4) + lane ----------------
  const int row = 32 * (warp & 3) + lane;
  const int my_r = row / G, my_g = row % G;
  float* xchg = reinterpret_cast<float*>(sm + kOffXchg);
  float qv[32];
  if (tid < 512) {  // (sixteen warps: four per lane quadrant, 32 dims each)
    const int part = warp >> 2;
    float qmax = 0.f;
    if (my_r < nrows) {
      const float4* src = reinterpret_cast<const float4*>(
          p.q_rot + ((int64_t)(lr0 + my_r) * sh.Hq + kvh * G + my_g) * kD + 32 * part);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 x = src[i];
        qv[4 * i] = x.x; qv[4 * i + 1] = x.y; qv[4 * i + 2] = x.z; qv[4 * i + 3] = x.w;
      }
#pragma unroll
      for (int i = 0; i < 32; ++i) qmax = fmaxf(qmax, fabsf(qv[i]));
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) qv[i] = 0.f;
    }
    xchg[part * 128 + row] = qmax;
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();  // the tensor-memory address, the table and the partial maxima are in place
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = s_tmem;
  const uint32_t lane_base = tmem + ((uint32_t)(32 * (warp & 3)) << 16);
  const float qmax = fmaxf(fmaxf(xchg[row], xchg[128 + row]), fmaxf(xchg[256 + row], xchg[384 + row]));
  // max|q| * sm_scale * log2(e) / alpha_k: the factor between a stored dot product and the score in
  // the log2 domain (at least the smallest normal number, so that a hidden score, -inf, times it stays -inf)
  const float qscale = fmaxf(qmax * (a.scale_log2e / a.lut_scale_k), 1.17549435e-38f);
  if (tid < 512) {
    const int part = warp >> 2;
    const float inv = qmax > 0.f ? 1.f / qmax : 0.f;
#pragma unroll
    for (int c = 0; c < 2; ++c) {  // 16 dims = 8 columns at a time
      uint32_t hi[8], lo[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float x0 = qv[16 * c + 2 * e] * inv, x1 = qv[16 * c + 2 * e + 1] * inv;
        const float h0 = __half2float(__float2half_rn(x0)), h1 = __half2float(__float2half_rn(x1));
        hi[e] = pack_h2(h0, h1);
        lo[e] = pack_h2(x0 - h0, x1 - h1);
      }
      tmem_st8_nowait(lane_base + kColQ + 16 * part + 8 * c, hi);
      if (!FAST) tmem_st8_nowait(lane_base + kColQlo + 16 * part + 8 * c, lo);
    }
    tmem_st_wait();
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();  // Q is in tensor memory; the exchange area is free again
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  // ---- softmax threads: row = TMEM lane = 32 * (warp & 3) + lane, column group = warp >> 2 -----------
  const bool smx = tid < kSmx;
  const int qt = (warp >> 2) % kTPR;  // which kCols score columns / kOCols output columns of the row
  const bool row_live = smx && my_r < nrows;
  // the threads of a row sit in warps w, w + 4, ...: a named barrier per such group of warps
  auto pair_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(1 + (warp & 3)), "n"(32 * kTPR) : "memory"); };
  const int kv_lo = row_live ? p.kv_start[lr0 + my_r] : 0;
  const int kv_hi = row_live ? p.kv_end[lr0 + my_r] : 0;
  // keys the block needs: rows are in query order, ranges move forward with the row
  const int blk_lo = p.kv_start[lr0], blk_hi = p.kv_end[lr0 + nrows - 1];
  const int t_first = blk_hi > blk_lo ? (blk_lo / kBN) * kBN : 0;
  const int n_tiles = blk_hi > blk_lo ? (blk_hi - t_first + kBN - 1) / kBN : 0;
  const int32_t* bt = a.block_table + (int64_t)p.row_seq[lr0] * a.bt_stride;
  const RowLayout lay = row_layout(sh.Hkv, kD);
  const int x_idx = lay.k_idx + kvh * 64, x_nrm = (lay.k_norm + kvh * 4) & ~15;
  const int n_sub = (lay.k_norm + kvh * 4) & 15;
  const int bs_mask = a.block_size - 1, bs_shift = __ffs(a.block_size) - 1;

  // one lane issues the boxes of tile j into stage j & 1: 4 pages x (indices K+V, norms K+V)
  // block ids of the four pages of tile j (read ahead of the copy issue: a global round trip)
  auto load_blks = [&](int j, int (&blk)[4]) {
    const int t0 = t_first + j * kBN;
#pragma unroll
    for (int pg = 0; pg < 4; ++pg) {
      const int pos = t0 + 16 * pg;
      // A volatile load straight into its register, from a clamped address instead of under a
      // condition: the ids are used an iteration later; an ordinary load gets moved down to its use, and
      // a select after the load makes the warp wait a global round trip right here, in every iteration.
      // (Pages past the block's last key are never issued, whatever id is read for them.)
      const int pos_c = min(pos, max(blk_hi - 1, 0));
      asm volatile("ld.global.nc.s32 %0, [%1];" : "=r"(blk[pg]) : "l"(bt + (pos_c >> bs_shift)));
    }
  };
  auto issue_tile = [&](int j, const int (&blks)[4]) {
    const uint32_t st = base + kOffStage + (uint32_t)(j & 1) * kStageBytes, bar = bar_t0 + 8 * (j & 1);
    const int t0 = t_first + j * kBN;
    int npages = 0;
#pragma unroll
    for (int pg = 0; pg < 4; ++pg) npages += (t0 + 16 * pg < blk_hi) ? 1 : 0;
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(npages * 2560) : "memory");
#pragma unroll
    for (int pg = 0; pg < 4; ++pg) {
      const int pos = t0 + 16 * pg;
      if (pos < blk_hi) {
        tma_load_4d(st + pg * 2048, &tm_idx, x_idx, pos & bs_mask, 0, blks[pg], bar);
        tma_load_4d(st + 8192 + pg * 512, &tm_norm, x_nrm, pos & bs_mask, 0, blks[pg], bar);
      }
    }
  };

  // ---- dequantise tile j (its packed stage has landed) into buffer j & 1: 512 items
  //      (K or V, token, 16-byte segment) spread over threads t of nt; norms by the first 64 --------
  // (item_lo, item_hi): items [0, 256) are the K half of the tile, [256, 512) the V half
  auto dequant_tile = [&](int j, int t, int nt, int item_lo, int item_hi) {
    const unsigned char* stg = sm + kOffStage + (j & 1) * kStageBytes;
    const uint32_t kv_off = (uint32_t)(j & 1) * 16384u;
    for (int item = item_lo + t; item < item_hi; item += nt) {
      // 32 consecutive items = 8 tokens x 4 segments; a quarter warp takes 4 tokens x the 2 segments of
      // one K-block, so that its eight 16-byte stores below (chunk ^ (token & 7)) fall into eight
      // different bank groups (token-major order made every store a two-way conflict)
      const int r8 = item & 7, q4 = (item >> 3) & 3;
      const int u = item >> 8, tok = ((item >> 5) & 7) * 8 + 4 * (q4 & 1) + (r8 & 3), seg = (r8 >> 2) + 2 * (q4 >> 1);
      const uint4 pk = *reinterpret_cast<const uint4*>(stg + (tok >> 4) * 2048 + u * 1024 + (tok & 15) * 64 + seg * 16);
      const uint32_t* lut = reinterpret_cast<const uint32_t*>(sm + kOffLut) + u * 256 * kLutCopies + lane;
      const uint32_t w[4] = {pk.x, pk.y, pk.z, pk.w};
      unsigned char* dst = sm + (u ? kOffV : kOffK) + kv_off + (seg >> 1) * 8192;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t x = w[c];
        const uint4 o = make_uint4(lut[(x & 255) * kLutCopies], lut[((x >> 8) & 255) * kLutCopies],
                                   lut[((x >> 16) & 255) * kLutCopies], lut[(x >> 24) * kLutCopies]);
        *reinterpret_cast<uint4*>(dst + swz(tok, (seg & 1) * 4 + c)) = o;
      }
    }
    if (item_lo == 0 && t < 64) {
      const unsigned char* nb = stg + 8192 + (t >> 4) * 512 + (t & 15) * 16 + n_sub;
      const float kn = *reinterpret_cast<const float*>(nb), vn = *reinterpret_cast<const float*>(nb + 256);
      float* ns = reinterpret_cast<float*>(sm + kOffNorm) + (j & 1) * 192;
      ns[t] = kn;
      ns[64 + t] = vn;
      ns[128 + t] = fmaxf(lg2_approx(vn), -30.f);
    }
  };
  // one page of tile j by the calling thread; the thread with `first` also posts the byte count of
  // the whole tile (the stage's barrier has one pending arrival, that one: bytes that land before it
  // cannot complete the phase)
  auto issue_page = [&](int j, int pg, int blk, bool first) {
    const uint32_t st = base + kOffStage + (uint32_t)(j & 1) * kStageBytes, bar = bar_t0 + 8 * (j & 1);
    const int t0 = t_first + j * kBN;
    if (first) {
      int npages = 0;
#pragma unroll
      for (int q = 0; q < 4; ++q) npages += (t0 + 16 * q < blk_hi) ? 1 : 0;
      asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(npages * 2560) : "memory");
    }
    const int pos = t0 + 16 * pg;
    if (pos < blk_hi) {
      tma_load_4d(st + pg * 2048, &tm_idx, x_idx, pos & bs_mask, 0, blk, bar);
      tma_load_4d(st + 8192 + pg * 512, &tm_norm, x_nrm, pos & bs_mask, 0, blk, bar);
    }
  };
  // descriptors of the operand regions; a byte offset inside a region adds offset / 16 to the
  // address field (all regions lie below 256 KB, the sum never carries into the other fields)
  const uint64_t d_k = desc_kmajor(base + kOffK), d_v = desc_mnmajor(base + kOffV, 8192);
  auto issue_s = [&](int j) {  // S = Q K~^T of tile j (one thread)
    const uint64_t dk = d_k + (uint64_t)((j & 1) * (16384 >> 4));
#pragma unroll
    for (int kb = 0; kb < 2; ++kb)
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const uint64_t db = dk + (uint64_t)((kb * 8192 + 32 * s) >> 4);
        const uint32_t qo = (uint32_t)(32 * kb + 8 * s);  // dims 64 kb + 16 s ...: two per column
        if (!FAST) mma_f16_ta(tmem + kColS + 64 * (j & 1), tmem + kColQlo + qo, db, kDescS, (kb | s) ? 1u : 0u);
        mma_f16_ta(tmem + kColS + 64 * (j & 1), tmem + kColQ + qo, db, kDescS, (FAST && !(kb | s)) ? 0u : 1u);
      }
    mma_commit(bar_s0 + 8 * (j & 1));  // one barrier per S buffer: a waiter can never be two phases behind
  };

  float m_run = -CUDART_INF_F, l_run = 0.f;
  bool o_zero = true;  // the O accumulator holds nothing yet (first PV overwrites)
  // ---- pipeline fill: tiles 0 and 1 in flight, tile 0 dequantised by everybody, S_0 issued ---------
  if (n_tiles > 0) {
    if (warp == kCopyWarp && elect_one_sync()) {
      int b0[4], b1[4];
      load_blks(0, b0);
      if (n_tiles > 1) load_blks(1, b1);
      issue_tile(0, b0);
      if (n_tiles > 1) issue_tile(1, b1);
    }
    const bool ok0 = bar_wait_bounded(bar_t0, 0u);
    dequant_tile(0, tid, kThreads, 0, 512);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    if (!ok0) s_info[3] = 1;
    __syncthreads();
    if (!s_info[3] && warp == kIssueWarp && elect_one_sync()) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      issue_s(0);
    }
  }

  int blk_next[4] = {0, 0, 0, 0};  // (copy warp) pages of the tile after next
  if (warp >= kCopyWarp - 3 && n_tiles > 2) load_blks(2, blk_next);
  // ---- per tile: warps 0-7 turn S_j into P_j while warps 8-15 dequantise tile j+1 and issue S_{j+1};
  //      then one thread issues O += P_j V~_j --------------------------------------------------------------
  bool gave_up = n_tiles > 0 && s_info[3] != 0;  // a bounded wait ran out somewhere in the block
  for (int j = 0; j < n_tiles && !gave_up; ++j) {
    const int t0 = t_first + j * kBN;
    bool ok = true;
    PF_STAMP(j, 0);
    if (!smx) {
      if (j + 1 < n_tiles) {
        // K~ buffer (j+1) & 1, its norms and S buffer (j+1) & 1 were last used for tile j-1, whose
        // scores the softmax warps consumed before the block barrier that ended the previous iteration
        ok = bar_wait_bounded(bar_t0 + 8 * ((j + 1) & 1), (uint32_t)(((j + 1) >> 1) & 1));
        PF_STAMP(j, 1);
        dequant_tile(j + 1, tid - kSmx, kDeq, 0, 256);  // keys and norms
        PF_STAMP(j, 2);
        // S_{j+1} goes into the other S buffer as soon as its K~ is in place: the softmax warps
        // find it ready when they finish tile j
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        asm volatile("bar.sync 5, %0;" ::"n"(kDeq) : "memory");
        const bool okw = __all_sync(0xffffffffu, ok);
        if (okw && warp == kIssueWarp && elect_one_sync()) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          issue_s(j + 1);
        }
        PF_STAMP(j, 3);
        // The packed stage of tile j was dequantised during the previous iteration: tile j + 2 goes into
        // it, most of an iteration before its turn (its page ids were read an iteration ago; those of
        // tile j + 3 are read after the values).  Issuing the eight copies takes the thread 1 000 - 2 000 cycles: here
        // they delay only its warp's share of the values; before the keys they would delay S_{j+1}.
        // Four warps issue one page each: a copy instruction costs its thread ~190 cycles.
        if (warp >= kCopyWarp - 3) {
          const int pg = warp - (kCopyWarp - 3);
          if (j + 2 < n_tiles && elect_one_sync()) issue_page(j + 2, pg, blk_next[pg], pg == 0);
          __syncwarp();
        }
        // the values of tile j + 1 (only O += P V~ of the next iteration reads them): V~ buffer
        // (j+1) & 1 was read by the MMAs of tile j-1
        if (j >= 1) ok = bar_wait_bounded(bar_o, (uint32_t)((j - 1) & 1)) && ok;
        PF_STAMP(j, 4);
        dequant_tile(j + 1, tid - kSmx, kDeq, 256, 512);
        PF_STAMP(j, 5);
        // (page ids of the tile after that: issued here, they cost the warp nothing before the barrier)
        if (warp >= kCopyWarp - 3 && j + 3 < n_tiles) load_blks(j + 3, blk_next);
      }
    } else {
      ok = __all_sync(0xffffffffu, bar_wait_bounded(bar_s0 + 8 * (j & 1), (uint32_t)((j >> 1) & 1)));
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      PF_STAMP(j, 1);
      const float* ns = reinterpret_cast<const float*>(sm + kOffNorm) + (j & 1) * 192 + kCols * qt;
      // sc[i] = dot product of column i times its key norm (-inf = not visible); the score in the log2
      // domain is sc[i] * qscale.  Tiles strictly inside the visible range of every row of the warp
      // take the short path without per-element masks.
      float sc[kCols];
      float mt = -CUDART_INF_F;
      const bool inner = __all_sync(0xffffffffu, ok && row_live && t0 >= kv_lo && t0 + kBN <= kv_hi);
      // 16 columns at a time (short register lifetimes); the second load is in flight while the first
      // half is processed
      constexpr int NH = kCols / 16;
      uint32_t vbuf[NH][16];
      if (ok) {
        tmem_ld16(lane_base + kColS + 64 * (j & 1) + kCols * qt, vbuf[0]);
        if (NH == 2) tmem_ld16_nowait(lane_base + kColS + 64 * (j & 1) + kCols * qt + 16, vbuf[NH - 1]);
      }
#pragma unroll
      for (int hh = 0; hh < NH; ++hh) {
        if (hh == 1) tmem_ld_wait16(vbuf[NH - 1]);
        uint32_t (&v)[16] = vbuf[hh];
        const float4* kn4 = reinterpret_cast<const float4*>(ns + 16 * hh);
        const float4* lg4 = reinterpret_cast<const float4*>(ns + 128 + 16 * hh);
        if (inner) {
#pragma unroll
          for (int i4 = 0; i4 < 4; ++i4) {
            const float4 kn = kn4[i4], lg = lg4[i4];
            const float kk[4] = {kn.x, kn.y, kn.z, kn.w}, ll[4] = {lg.x, lg.y, lg.z, lg.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float s = __uint_as_float(v[4 * i4 + e]) * kk[e];
              sc[16 * hh + 4 * i4 + e] = s;
              mt = fmaxf(mt, fmaf(s, qscale, ll[e]));
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int pos = t0 + kCols * qt + 16 * hh + i;
            const bool vis = ok && row_live && pos >= kv_lo && pos < kv_hi;
            const float s = vis ? __uint_as_float(v[i]) * ns[16 * hh + i] : -CUDART_INF_F;
            sc[16 * hh + i] = s;
            mt = fmaxf(mt, vis ? fmaf(s, qscale, ns[128 + 16 * hh + i]) : -CUDART_INF_F);
          }
        }
      }
      // the row's maximum over both halves (the decisions below must agree in its two threads)
      PF_STAMP(j, 2);
      xchg[qt * 128 + row] = mt;
      pair_sync();
#pragma unroll
      for (int o = 1; o < kTPR; ++o) mt = fmaxf(mt, xchg[((qt + o) % kTPR) * 128 + row]);
      PF_STAMP(j, 3);
      // P and O are still in use by the MMAs of tile j-1
      if (j >= 1) ok = __all_sync(0xffffffffu, bar_wait_bounded(bar_o, (uint32_t)((j - 1) & 1))) && ok;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      PF_STAMP(j, 4);
      // lazily updated reference: moves only when a score (shifted by log2 of its value norm)
      // exceeds it by more than 2^8; then this row of O is rescaled in tensor memory
      const bool bump = mt > m_run + 8.f;
      if (__any_sync(0xffffffffu, bump)) {
        const float alpha = bump ? (m_run == -CUDART_INF_F ? 0.f : ex2_approx(m_run - mt)) : 1.f;
        if (bump) { m_run = mt; l_run *= alpha; }
        if (!o_zero && ok) {
#pragma unroll
          for (int q = 0; q < kOCols / 16; ++q) {  // this thread's share of the row's 128 columns
            uint32_t v[16];
            tmem_ld16(lane_base + kColO + kOCols * qt + 16 * q, v);
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st16(lane_base + kColO + kOCols * qt + 16 * q, v);
          }
        }
      }
      const float m_neg = m_run == -CUDART_INF_F ? 0.f : -m_run;
      float lsum = 0.f;
      const float4* vn4 = reinterpret_cast<const float4*>(ns + 64);
      // (two instances of the loop: inside the visible range of every row of the warp there is nothing
      //  to select, which saves two instructions per column)
      auto exp_phase = [&](auto inner_tag) {
        constexpr bool INNER = decltype(inner_tag)::value;
#pragma unroll
        for (int c = 0; c < kCols / 16; ++c) {  // 16 tokens = 8 columns of P at a time
          uint32_t h[8], lw[8];
#pragma unroll
          for (int e4 = 0; e4 < 4; ++e4) {
            const float4 va = vn4[4 * c + e4];
            const float vv[4] = {va.x, va.y, va.z, va.w};
#pragma unroll
            for (int e = 0; e < 2; ++e) {
              const int t = 16 * c + 4 * e4 + 2 * e;
              const float e0 = ex2_approx(fmaf(sc[t], qscale, m_neg)), e1 = ex2_approx(fmaf(sc[t + 1], qscale, m_neg));
              lsum += e0 + e1;
              // (a hidden column has e = 0; its value norm may be anything, so select instead of multiply)
              const float v0 = (INNER || sc[t] != -CUDART_INF_F) ? e0 * vv[2 * e] : 0.f;
              const float v1 = (INNER || sc[t + 1] != -CUDART_INF_F) ? e1 * vv[2 * e + 1] : 0.f;
              const __half2 hp = __floats2half2_rn(v0, v1);
              const float2 hf2 = __half22float2(hp);
              h[2 * e4 + e] = *reinterpret_cast<const uint32_t*>(&hp);
              if (!FAST) lw[2 * e4 + e] = pack_h2(v0 - hf2.x, v1 - hf2.y);  // the fp16 rounding of the weights is recovered by a second term
            }
          }
          tmem_st8_nowait(lane_base + kColP + (kCols / 2) * qt + 8 * c, h);
          if (!FAST) tmem_st8_nowait(lane_base + kColPlo + (kCols / 2) * qt + 8 * c, lw);
        }
      };
      if (inner) exp_phase(std::true_type{});
      else exp_phase(std::false_type{});
      tmem_st_wait();
      l_run += lsum;  // (this thread's half of the row sum)
      PF_STAMP(j, 5);
    }
    if (!smx) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // (the dequantised values)
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    gave_up = __syncthreads_or(!ok) != 0;  // (the flag travels with the barrier: no shared-memory read)
    PF_STAMP(j, 7);
    if (gave_up) break;
    if (warp == kIssueWarp && elect_one_sync()) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      const uint64_t dvb = d_v + (uint64_t)((j & 1) * (16384 >> 4));
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        const uint64_t dv = dvb + (uint64_t)((2048 * s) >> 4);
        if (!FAST) mma_f16_ta(tmem + kColO, tmem + kColPlo + 8 * s, dv, kDescO, (!o_zero || s) ? 1u : 0u);
        mma_f16_ta(tmem + kColO, tmem + kColP + 8 * s, dv, kDescO, (FAST && o_zero && !s) ? 0u : 1u);
      }
      mma_commit(bar_o);
    }
    PF_STAMP(j, 8);
    o_zero = false;
  }
  if (gave_up && tid == 0) s_info[3] = 1;
  if (n_tiles > 0 && !gave_up) {  // the last tile's MMAs
    if (!bar_wait_bounded(bar_o, (uint32_t)((n_tiles - 1) & 1))) s_info[3] = 1;
  }
  __syncthreads();

  // ---- normalised rotated output + log-sum-exp, as one dense partial per (row, head) ------------
  const bool dead = s_info[3] != 0;
  if (smx) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    xchg[qt * 128 + row] = l_run;  // the row sum = the shares of its threads
    pair_sync();
#pragma unroll
    for (int o = 1; o < kTPR; ++o) l_run += xchg[((qt + o) % kTPR) * 128 + row];
    const bool have = !dead && !o_zero && l_run > 0.f;
    const float inv = have ? 1.f / (a.lut_scale_v * l_run) : 0.f;
    const int64_t vec = row_live ? (int64_t)(lr0 + my_r) * sh.Hq + kvh * G + my_g : 0;
#pragma unroll
    for (int q = 0; q < kOCols / 32; ++q) {  // this thread's columns
      uint32_t v[32];
      if (!o_zero && !dead) {
        tmem_ld32(lane_base + kColO + kOCols * qt + 32 * q, v);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0u;
      }
      if (row_live) {
        float4* dst = reinterpret_cast<float4*>(p.part_o + vec * kD + kOCols * qt + 32 * q);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          dst[i] = make_float4(__uint_as_float(v[4 * i]) * inv, __uint_as_float(v[4 * i + 1]) * inv,
                               __uint_as_float(v[4 * i + 2]) * inv, __uint_as_float(v[4 * i + 3]) * inv);
      }
    }
    if (row_live && qt == 0)
      p.part_m[vec] = have ? (m_run + lg2_approx(l_run)) * 0.6931471805599453f : -CUDART_INF_F;
  }
  if (dead && tid == 0 && a.err_flag) atomicOr(a.err_flag, TQ4_DEV_TIMEOUT);
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ---- host side -------------------------------------------------------------------------------------
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
// dims (bytes of one half of a token row, tokens in a block, K/V half, blocks); box = 16 tokens x both halves
bool make_map(CUtensorMap* m, const AttnArgs& a, uint32_t box_bytes) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t half_bytes = (cuuint64_t)a.sh.Hkv * (a.sh.D / 2 + 4);
  const cuuint64_t dims[4] = {half_bytes, (cuuint64_t)a.block_size, 2, (cuuint64_t)a.num_blocks};
  const cuuint64_t strides[3] = {(cuuint64_t)a.cache_token_stride, half_bytes, (cuuint64_t)a.cache_block_stride};
  const cuuint32_t box[4] = {box_bytes, 16, 2, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<uint8_t*>(a.cache), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int G, bool FAST>
int launch_t(const AttnArgs& a, cudaStream_t st) {
  const int smem = (int)kSmemBytes + 1024;
  if (!ensure_dynamic_smem<prefill_tc_kernel<G, FAST>>(smem)) return TQ4_ERR_CUDA;
  CUtensorMap tm_idx, tm_norm;
  memset(&tm_idx, 0, sizeof(tm_idx));
  memset(&tm_norm, 0, sizeof(tm_norm));
  if (!make_map(&tm_idx, a, 64) || !make_map(&tm_norm, a, 16)) return TQ4_ERR_UNSUPPORTED;
  constexpr int RB = 128 / G;
  const unsigned blocks = (unsigned)((a.sh.rows + RB - 1) / RB + a.sh.num_seqs);  // upper bound
  if (launch_kernel(prefill_tc_kernel<G, FAST>, dim3(blocks, (unsigned)a.sh.Hkv), dim3(kThreads), (size_t)smem, st,
                    true, a, tm_idx, tm_norm) != cudaSuccess)
    return TQ4_ERR_CUDA;
  TQ4_CHECK_LAUNCH();
  return TQ4_OK;
}

}  // namespace

// Shapes and layouts the tensor-core prefill kernel covers (everything else streams).
bool prefill_tc_supported(const AttnArgs& a) {
  static const bool disabled = getenv("TQ4_NO_TC") != nullptr;
  const int G = a.sh.G;
  const RowLayout lay = row_layout(a.sh.Hkv, a.sh.D);
  return !disabled && a.sh.D == kD && (G == 1 || G == 2 || G == 4 || G == 8) && a.query_start_loc != nullptr &&
         (uintptr_t)a.cache % 16 == 0 && a.cache_block_stride % 16 == 0 && a.cache_token_stride % 16 == 0 &&
         a.block_size % 16 == 0 && a.block_size <= 256 && (a.block_size & (a.block_size - 1)) == 0 &&
         lay.v_idx % 16 == 0 && a.num_blocks < (1ll << 31) && encode_fn() != nullptr;
}

int launch_prefill_tc(const AttnArgs& a, cudaStream_t st, bool fast) {
  switch (a.sh.G) {
    case 1: return fast ? launch_t<1, true>(a, st) : launch_t<1, false>(a, st);
    case 2: return fast ? launch_t<2, true>(a, st) : launch_t<2, false>(a, st);
    case 4: return fast ? launch_t<4, true>(a, st) : launch_t<4, false>(a, st);
    case 8: return fast ? launch_t<8, true>(a, st) : launch_t<8, false>(a, st);
  }
  return TQ4_ERR_UNSUPPORTED;
}

}  // namespace tq4

#ifdef TQ4_TRACE
extern "C" int tq4_prefill_trace_read(long long* out) {
  return cudaMemcpyFromSymbol(out, tq4::g_ptrace, sizeof(long long) * 4 * 64 * 16) == cudaSuccess ? 0 : 1;
}
#endif
