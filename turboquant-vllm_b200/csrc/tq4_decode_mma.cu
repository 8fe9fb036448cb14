// Paged TQ4 attention, tensor-core LUT kernel (the HBM-bound decode path).
//
// One warp streams 16-token tiles of one KV head for up to 8 query heads of its GQA group.
// Both products run on mma.sync.m16n8k16 (f16 operands, f32 accumulate) in TRANSPOSED form,
// so the packed cache bytes feed the A operand and the tiny query/probability matrices are
// the B operand (N = 8 columns = 4 heads x {hi, lo} fp16 split terms, which makes the
// query- and probability-side rounding error-free to ~2^-22):
//     S^T[16 tok x 8]   = K[16 tok x 16 dims]    * Qsplit^T[16 dims x 8]      (D/16 k-steps)
//     O^T[16 dims x 8] += V^T[16 dims x 16 tok]  * Psplit^T[16 tok x 8]       (D/16 m-blocks)
// Dequantisation is ONE shared-memory load per packed byte: a 256-entry table maps a byte
// (two nibbles) to a half2 of two centroids, replicated per lane so that every lane reads
// its own bank (conflict-free); the load address is formed by a single PRMT that drops the
// byte into bits 8..15 of a per-lane base (the table is 64 KB-aligned in the shared window).
// For K a byte is (even dim, odd dim) of one token = one A register.  For V the A register
// needs (token j, token j+1) of one dim, so bytes of two adjacent tokens are re-paired with
// two LOP3s per 8 nibbles before the lookup.  Table entries are fp16(alpha * centroid) with a
// per-codebook alpha (tq4_lut_scale.h) that puts all centroid magnitudes near fp16 grid points;
// 1/alpha is folded into the fp32 score scale and the output.  Norms are factored out: scores are scaled by
// knorm in fp32, probabilities by vnorm before the split.
//
// Work: the tile stream of a call is cut into one contiguous span per warp; a warp walks the
// (query row, span) segments of its span and writes one partial (m, l, O) per segment.
//
// Data movement: a per-warp shared-memory ring of two stages, one pair of tiles each.  With TMA
// (the usual case) one elected lane issues the pair's box copies (two 4-D boxes per tile when the
// K and V halves of a token row are 16-byte aligned, a wider-V 3-D scheme or one whole-row box
// otherwise) onto the stage's mbarrier; every wait is bounded.  Layouts TMA cannot address fall
// back to per-thread cp.async of exactly the bytes each thread consumes.  Tiles are read back
// with 16/8-byte shared loads at compile-time offsets; a token permutation plus the 64-byte TMA
// swizzle keep them free of bank conflicts.
#include <cuda.h>
#include <math_constants.h>

#include <cstdlib>
#include <cstring>

#include "tq4_attention.cuh"

namespace tq4 {

namespace {

constexpr uint32_t kTableBytes = 65536;

// Timeline aid for tuning builds (-DTQ4_TRACE): lane 0 of every warp stamps %globaltimer at a few
// points into a buffer read back with tq4_trace_read.  Compiled out of the shipped library.
#ifdef TQ4_TRACE
__device__ long long g_trace[160 * 16 * 16];
#define TQ4_STAMP(i)                                                                             \
  do {                                                                                           \
    if ((threadIdx.x & 31) == 0) {                                                               \
      long long t__;                                                                             \
      asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t__));                                    \
      g_trace[((blockIdx.x % 160) * 16 + (threadIdx.x >> 5)) * 16 + (i)] = t__;                   \
    }                                                                                            \
  } while (0)
#else
#define TQ4_STAMP(i) do {} while (0)
#endif
constexpr int kStages = 2;  // ring stages per warp, one PAIR of 16-token tiles each

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

template <int BYTE>
__device__ __forceinline__ uint32_t lut(uint32_t w, uint32_t lanebase) {
  uint32_t addr, v;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(addr) : "r"(w), "r"(lanebase), "n"(0x7604 | (BYTE << 4)));
  asm("ld.shared.b32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}

__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// first MMA of an accumulation chain: C = 0 (no zero-initialised accumulator registers needed)
__device__ __forceinline__ void mma16816_zero(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2,
                                              uint32_t a3, uint32_t b0, uint32_t b1) {
  asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%10,%10,%10,%10};"
      : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t x) {
  uint32_t y;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(y) : "r"(x));
  return y;
}

__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// split x into fp16 hi + fp16 lo and pack (hi, lo) into one register
__device__ __forceinline__ uint32_t split_h2(float x) {
  const __half h = __float2half_rn(x);
  const __half l = __float2half_rn(x - __half2float(h));
  __half2 r = __halves2half2(h, l);
  return *reinterpret_cast<uint32_t*>(&r);
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

template <int BYTES>
__device__ __forceinline__ void cp_async(uint32_t dst, const uint8_t* src) {
  if (BYTES == 16)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
  else if (BYTES == 8)
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

template <int BYTES>
__device__ __forceinline__ void lds_words(uint32_t addr, uint32_t* out) {
  if (BYTES == 16)
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(out[0]), "=r"(out[1]), "=r"(out[2]), "=r"(out[3]) : "r"(addr));
  else if (BYTES == 8)
    asm volatile("ld.shared.v2.b32 {%0,%1}, [%2];" : "=r"(out[0]), "=r"(out[1]) : "r"(addr));
  else
    asm volatile("ld.shared.b32 %0, [%1];" : "=r"(out[0]) : "r"(addr));
}

// ---- mbarrier / TMA (bulk tensor copy) primitives; every wait is bounded ---------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
// Returns false if the phase did not complete within the iteration limit.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity) {
  for (int it = 0; it < (1 << 18); ++it)
    if (mbar_try_wait(bar, parity)) return true;
  return false;
}
// True in exactly one lane of a converged warp; tells the compiler that the guarded region is
// single-threaded, so bulk-copy instructions inside it need no per-thread serialisation loop.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
      : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int x, int y, int z,
                                            int w, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(map), "r"(x), "r"(y), "r"(z), "r"(w), "r"(bar)
      : "memory");
}
// shared-memory loads at base + compile-time offset (the offset lands in the instruction)
template <int BYTES, int IMM>
__device__ __forceinline__ void lds_imm(uint32_t base, uint32_t* out) {
  if (BYTES == 16)
    asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4+%5];"
                 : "=r"(out[0]), "=r"(out[1]), "=r"(out[2]), "=r"(out[3]) : "r"(base), "n"(IMM));
  else if (BYTES == 8)
    asm volatile("ld.shared.v2.b32 {%0,%1}, [%2+%3];" : "=r"(out[0]), "=r"(out[1]) : "r"(base), "n"(IMM));
  else
    asm volatile("ld.shared.b32 %0, [%1+%2];" : "=r"(out[0]) : "r"(base), "n"(IMM));
}

template <int D, bool ALIGNED>
struct MmaCfg {
  static constexpr int HALF = D / 2;
  static constexpr int KS = D / 16;         // k-steps of the K-side product
  static constexpr int KBY = D / 8;         // K bytes per thread per token
  static constexpr int KW = KBY / 4;        // ... as 32-bit words
  static constexpr int VBY = D / 16;        // V bytes per thread per token
  static constexpr int VW = VBY / 4;        // ... full words
  static constexpr int VH = (VBY % 4) / 2;  // ... plus one half-word (D = 96)
  static constexpr int MB = VBY;            // m-blocks of the V-side product
  static constexpr int DPT = D / 4;         // query dims held per thread
  // cp.async unit sizes (bytes) and counts
  static constexpr int UK = ALIGNED ? (KBY >= 16 ? 16 : KBY) : 4;
  static constexpr int NK = KBY / UK;
  static constexpr int UV = ALIGNED ? (4 * VW >= 16 ? 16 : 4 * VW) : 4;
  static constexpr int NV = (4 * VW) / UV;
  // per-warp bytes of one ring stage: K (2 tokens) + V (4 tokens: words + half-word unit) + norms
  static constexpr int kVTok = 32 * (4 * VW + 4 * VH);
  static constexpr int kOffK1 = 32 * KBY;
  static constexpr int kOffV = 64 * KBY;
  static constexpr int kOffN = kOffV + 4 * kVTok;
  static constexpr int kStageBytes = kOffN + 32 * 16;
  // TMA stage: K tile [16 tok][D/2] | V tile [16 tok][D/2] | K-norm tile [16][16 B] | V-norm tile
  // (VWIDE: the V box starts 0..12 bytes early, on a 16-byte boundary, and is 16 bytes wider)
  static constexpr int kTmaV = 16 * HALF;
  template <bool VWIDE> __host__ __device__ static constexpr int v_pitch() { return VWIDE ? HALF + 16 : HALF; }
  template <bool VWIDE> __host__ __device__ static constexpr int tma_kn() { return 16 * HALF + 16 * v_pitch<VWIDE>(); }
  template <bool VWIDE> __host__ __device__ static constexpr int tma_stage() { return tma_kn<VWIDE>() + 512; }
};


// =====================================================================================================
// Fused prologue (decode calls of at most kFusedMaxRows rows, head_dim <= 128): the attention kernel
// itself computes the tile plan and rotates the queries, so a decode step needs no kernel in front
// of it and no CTA waits for another.
//
//  * Plan: every warp scans the rows of the call (32 per step), sums their tile counts, derives the
//    tiles per span and writes the plan arrays of the chunks it owns; all CTAs write the same
//    values, each reads back only what it wrote itself (after a block barrier).
//  * Rotation: a CTA rotates exactly the query rows its own spans touch (all heads of its slice):
//    q_rot = q * Pi^T on mma.sync.m16n8k16 with both operands split into fp16 hi + lo terms
//    (hi*hi + hi*lo + lo*hi, fp32 accumulate: about 2^-21 relative).  Pi (times 2^8, so that the lo
//    terms stay normal numbers) sits in shared memory as two fp16 arrays in the 64 KB region that
//    afterwards holds the dequantisation table; each query vector is scaled by a power of two
//    into [1, 2) before its split.  Neighbouring CTAs that share a row compute the same values and
//    store the same bits.
// =====================================================================================================

template <int D>
struct RotCfg {
  static constexpr int KS = D / 16;                      // k-steps
  static constexpr int NBT = 2;                          // n-blocks (of 8 outputs) per task
  static constexpr int NQ = D / (8 * NBT);               // tasks along N: small tasks spread evenly over 16 warps
  static constexpr int PITCH = 2 * D + (D == 96 ? 32 : 0);  // bytes per row of a Pi half (fp16)
  static constexpr bool XOR = D != 96;                   // 8-byte chunks XOR-swizzled by 4 * (row & 3)
  static constexpr int LO_BASE = D * PITCH;              // the lo array follows the hi array
  static_assert(2 * D * PITCH <= (int)kTableBytes, "both fp16 halves of Pi fit the table region");
};

template <int D>
__device__ __forceinline__ uint32_t rot_chunk_off(int n, int kc) {  // byte offset of 8-byte chunk kc of row n
  using R = RotCfg<D>;
  return (uint32_t)(n * R::PITCH + ((R::XOR ? (kc ^ (4 * (n & 3))) : kc) << 3));
}

// fp16 hi / lo split of four floats -> (hi01, hi23, lo01, lo23)
__device__ __forceinline__ void split4(const float (&x)[4], uint32_t& h01, uint32_t& h23, uint32_t& l01,
                                       uint32_t& l23) {
  float h[4], l[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    h[i] = __half2float(__float2half_rn(x[i]));
    l[i] = x[i] - h[i];
  }
  h01 = pack_h2(h[0], h[1]); h23 = pack_h2(h[2], h[3]);
  l01 = pack_h2(l[0], l[1]); l23 = pack_h2(l[2], l[3]);
}

// Stage Pi * 2^8 as fp16 hi / lo arrays at shared address `tab` (all threads of the block).
template <int D>
__device__ __forceinline__ void stage_rotation_split(const float* __restrict__ rotation, uint32_t tab) {
  constexpr int N4 = D * D / 4;
  constexpr int kBatch = 8;  // 16-byte loads in flight per thread (Pi is L2-resident: one round trip per batch)
  for (int i0 = threadIdx.x; i0 < N4; i0 += kBatch * blockDim.x) {
    float4 x[kBatch];
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int i = i0 + u * blockDim.x;
      if (i < N4) x[u] = __ldg(reinterpret_cast<const float4*>(rotation) + i);
    }
#pragma unroll
    for (int u = 0; u < kBatch; ++u) {
      const int i = i0 + u * blockDim.x;
      if (i < N4) {
        const int n = i / (D / 4), kc = i - n * (D / 4);
        const float v[4] = {x[u].x * 256.f, x[u].y * 256.f, x[u].z * 256.f, x[u].w * 256.f};
        uint32_t h01, h23, l01, l23;
        split4(v, h01, h23, l01, l23);
        const uint32_t off = tab + rot_chunk_off<D>(n, kc);
        asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(off), "r"(h01), "r"(h23) : "memory");
        asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(off + RotCfg<D>::LO_BASE), "r"(l01), "r"(l23) : "memory");
      }
    }
  }
}

// The same in two phases for blocks that hold the whole matrix in one batch of loads (kPiBatch per
// thread): the loads are issued first, the plan is computed while they are in flight, then the
// values are split and stored.
constexpr int kPiBatch = 8;
template <int D>
__device__ __forceinline__ void pi_load(const float* __restrict__ rotation, float4 (&x)[kPiBatch]) {
#pragma unroll
  for (int u = 0; u < kPiBatch; ++u) {
    const int i = threadIdx.x + u * blockDim.x;
    if (i < D * D / 4) x[u] = __ldg(reinterpret_cast<const float4*>(rotation) + i);
  }
}
template <int D>
__device__ __forceinline__ void pi_store(const float4 (&x)[kPiBatch], uint32_t tab) {
#pragma unroll
  for (int u = 0; u < kPiBatch; ++u) {
    const int i = threadIdx.x + u * blockDim.x;
    if (i < D * D / 4) {
      const int n = i / (D / 4), kc = i - n * (D / 4);
      const float v[4] = {x[u].x * 256.f, x[u].y * 256.f, x[u].z * 256.f, x[u].w * 256.f};
      uint32_t h01, h23, l01, l23;
      split4(v, h01, h23, l01, l23);
      const uint32_t off = tab + rot_chunk_off<D>(n, kc);
      asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(off), "r"(h01), "r"(h23) : "memory");
      asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(off + RotCfg<D>::LO_BASE), "r"(l01), "r"(l23) : "memory");
    }
  }
}

// Visible key range of decode row r (the single query of sequence r + row_offset).
__device__ __forceinline__ void decode_row_range(const AttnArgs& a, int r, int& seq, int& start, int& end) {
  const int gr = r + a.sh.row_offset;
  seq = 0; start = 0; end = 0;
  if (gr < a.sh.num_seqs) {
    seq = gr;
    const int len = clamp_seq_len(a, max(0, __ldg(a.seq_lens + gr)));
    end = len;
    start = a.sliding_window > 0 ? max(0, len - a.sliding_window) : 0;
  }
}

__device__ __forceinline__ int warp_incl_scan(int v, int lane) {
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += up;
  }
  return v;
}

// Tiles of a row that sees keys [start, end).
__device__ __forceinline__ int row_tiles(int start, int end) {
  return end > start ? (end + kTileTokens - 1) / kTileTokens - start / kTileTokens : 0;
}

// What one warp knows about the plan of a decode call after scanning the sequence lengths once
// (registers only; nothing is read back from global memory).
struct WarpPlan {
  int total, tps;        // tiles of the call, tiles per span
  int r0, r0_t0, r0_slot;  // first row of the warp's span (-1: the span is empty), its first tile, its first partial slot
  int r_a, r_b;          // rows holding the first and the last tile of the CTA's tile range (-1: empty range)
  int t_a, t_b;          // the CTA's tile range
  bool rb_ends;          // row r_b's last tile lies inside the range (rows r_a .. r_b - 1 always end inside)
};

// The plan of a decode call as one warp needs it.  Code that runs once per launch pays for every
// instruction it fetches, so this is two short rolled loops over chunks of 32 rows: the first sums
// the tile counts, the second scans them (the sequence lengths are read again; they sit in L1 by
// then) and derives the partial slots per row and the rows that hold the tiles the warp and its
// CTA start and end with.  CTA 0 also stores the slot prefix the merge kernel reads after this
// kernel has finished.
__device__ __forceinline__ WarpPlan fused_plan(const AttnArgs& a, int warp, int n_warps, int lane,
                                               int span, int span_first, int span_count) {
  const AttnShape& sh = a.sh;
  const int rows = sh.rows, n_chunks = (rows + 31) >> 5;
  auto tiles_of = [&](int r) -> int {
    int seq, start = 0, end = 0;
    if (r < rows) decode_row_range(a, r, seq, start, end);
    return row_tiles(start, end);
  };
  int local = 0, longest = 0;
#pragma unroll 4
  for (int ch = 0; ch < n_chunks; ++ch) {  // (independent loads, in flight together)
    const int nt = tiles_of(ch * 32 + lane);
    local += nt;
    longest = max(longest, nt);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    local += __shfl_xor_sync(0xffffffffu, local, o);
    longest = max(longest, __shfl_xor_sync(0xffffffffu, longest, o));
  }
  WarpPlan wp;
  wp.total = local;
  wp.tps = tiles_per_span(wp.total, sh.span_ctas, longest);
  const int T_a = (int)min((long long)span_first * wp.tps, (long long)wp.total);
  const int T_b = (int)min((long long)wp.total, (long long)T_a + (long long)span_count * wp.tps);
  const long long T_w = (long long)span * wp.tps;  // first tile of the warp's own span
  wp.t_a = T_a;
  wp.t_b = T_b;
  wp.r0 = wp.r_a = wp.r_b = -1;
  wp.r0_t0 = wp.r0_slot = 0;
  wp.rb_ends = false;
  int run_t = 0, run_s = 0;
#pragma unroll 1
  for (int ch = 0; ch < n_chunks; ++ch) {
    const int nt = tiles_of(ch * 32 + lane);
    const int incl_t = warp_incl_scan(nt, lane);
    const int b = run_t + incl_t - nt, e = b + nt;
    const int ns = nt > 0 ? (e - 1) / wp.tps - b / wp.tps + 1 : 0;
    const int incl_s = warp_incl_scan(ns, lane);
    const int pre_s = run_s + incl_s - ns;
    if (blockIdx.x == 0 && ch % n_warps == warp && ch * 32 + lane < rows)
      a.plan.slot_base[ch * 32 + lane] = pre_s;
    // rows that hold: the warp's first tile, the CTA's first tile, the CTA's last tile
    const unsigned mw = __ballot_sync(0xffffffffu, nt > 0 && b <= T_w && T_w < e);
    const unsigned ma = __ballot_sync(0xffffffffu, T_a < T_b && nt > 0 && b <= T_a && T_a < e);
    const unsigned mb = __ballot_sync(0xffffffffu, T_a < T_b && nt > 0 && b < T_b && T_b <= e);
    if (mw) {
      wp.r0 = ch * 32 + __ffs(mw) - 1;
      wp.r0_t0 = __shfl_sync(0xffffffffu, b, __ffs(mw) - 1);
      wp.r0_slot = __shfl_sync(0xffffffffu, pre_s, __ffs(mw) - 1);
    }
    if (ma) wp.r_a = ch * 32 + __ffs(ma) - 1;
    if (mb) {
      wp.r_b = ch * 32 + __ffs(mb) - 1;
      wp.rb_ends = __shfl_sync(0xffffffffu, e, __ffs(mb) - 1) == T_b;
    }
    run_t += __shfl_sync(0xffffffffu, incl_t, 31);
    run_s += __shfl_sync(0xffffffffu, incl_s, 31);
  }
  if (blockIdx.x == 0 && warp == 0 && lane == 0) a.plan.slot_base[rows] = run_s;
  return wp;
}

// Four consecutive elements e0 .. e0 + 3 of a query vector as floats.
__device__ __forceinline__ void load_q4(const void* q, int dtype, int64_t idx, bool vec_ok, float (&x)[4]) {
  if (vec_ok) {
    if (dtype == TQ4_F32) {
      const float4 v = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(q) + idx));
      x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    } else {
      const uint2 v = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const uint16_t*>(q) + idx));
      if (dtype == TQ4_F16) {
        const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
        const float2 f1 = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
        x[0] = f0.x; x[1] = f0.y; x[2] = f1.x; x[3] = f1.y;
      } else {
        x[0] = __uint_as_float(v.x << 16); x[1] = __uint_as_float(v.x & 0xFFFF0000u);
        x[2] = __uint_as_float(v.y << 16); x[3] = __uint_as_float(v.y & 0xFFFF0000u);
      }
    }
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i) x[i] = load_as_float(q, dtype, idx + i);
  }
}

// Rotation work of a CTA, on mma.sync (see the header of this section).  The vectors of a CTA are
//  * q rows [r_a, r_b] x heads [h0, h0 + nh), rotated into the q_rot scratch, and
//  * with `w` (a decode step's cache write) the K and V vectors of the new token of every row of
//    [r_a, r_b] whose LAST tile lies in the CTA's tile range, for the KV heads [kvh0, kvh0 + nkv):
//    norm (summed in the order of the compress kernels, so the stored norms are bit-identical to
//    theirs), x / (norm + 1e-10), rotation, bucketize, nibble pack, stored at the token's slot.  The
//    CTA that reads a row's last tile is the one that writes it, so a block barrier (plus the
//    generic -> async proxy fence) orders the write before the read.
// They are handled in GROUPS of 16.  fused_prep_group (one warp per group) turns a group into the
// A operand of the product -- 16 x D fp16 hi and lo tiles in the warp's (still idle) ring memory,
// each vector scaled by a power of two into [1, 2) -- plus 16 bytes of bookkeeping per vector;
// fused_mma_task multiplies (group, 16 output coordinates) tasks, handed out to all warps round
// robin.  Both are short rolled loops: code that runs once per launch costs its instruction
// fetches.  Lane (g, c) owns, per k-step s, the four contiguous elements 16 s + 4 c .. + 3 of
// vectors g and g + 8 (the k order inside a step is a permutation applied to both operands).
struct RotRows {
  int r_a, r_b;      // query rows of the CTA
  bool rb_ends;      // row r_b's last tile belongs to the CTA (rows before it always end inside)
  int h0, nh;        // query heads of the CTA's slice
  int kvh0, nkv;     // KV heads of the CTA's slice
  int n_q, n_vec;    // query vectors, all vectors (queries first, then K / V vectors of the new tokens)
};
// per-vector bookkeeping word: where the result goes
constexpr unsigned long long kRowInvalid = 1ull << 63, kRowWrite = 1ull << 62, kRowV = 1ull << 61;
constexpr unsigned long long kRowOffMask = (1ull << 61) - 1;
template <int D>
struct GroupMem {  // byte offsets inside a warp's ring memory
  static constexpr int kHalf = 16 * RotCfg<D>::PITCH;  // one 16 x D fp16 tile
  static constexpr int kInfo = 2 * kHalf;              // 16 x {u64 where, f32 1 / scale, f32 norm}
  static constexpr int kBytes = kInfo + 16 * 16;
};

template <int D>
__device__ __forceinline__ void fused_prep_group(const AttnArgs& a, const CompressArgs& w, bool has_write,
                                                 const RotRows& rr, int group, uint32_t mem, int lane) {
  using R = RotCfg<D>;
  const AttnShape& sh = a.sh;
  const int g = lane >> 2, c = lane & 3;
  const RowLayout lay = row_layout(sh.Hkv, D);
#pragma unroll 1
  for (int hf = 0; hf < 2; ++hf) {  // vector g, then vector g + 8 of the group
    const int row = g + 8 * hf, v = group * 16 + row;
    unsigned long long where = kRowInvalid;
    const void* src_ptr = nullptr;
    int src_dtype = a.q_dtype;
    int64_t base = 0, ts = a.q_token_stride, hs = a.q_head_stride;
    if (v < rr.n_q) {
      const int ri = v / rr.nh, h = rr.h0 + (v - ri * rr.nh);
      const int r = rr.r_a + ri;
      where = (unsigned long long)(((int64_t)r * sh.Hq + h) * D);
      src_ptr = a.q;
      base = ((int64_t)r + sh.row_offset) * ts + (int64_t)h * hs;
    } else if (v < rr.n_vec) {
      const int wi = v - rr.n_q;
      const int ri = wi / (2 * rr.nkv), rem = wi - ri * (2 * rr.nkv);
      const int src = rem >= rr.nkv ? 1 : 0, kvh = rr.kvh0 + rem - src * rr.nkv;
      const int r = rr.r_a + ri, tok = r + sh.row_offset;
      if (tok < w.n_tokens && tok < w.n_slots) {
        // the loads below do not depend on one another: one memory round trip
        int seq, kv_start, kv_end;
        decode_row_range(a, r, seq, kv_start, kv_end);
        const int64_t slot = __ldg(w.slot_mapping + tok);
        const int pos = max(kv_end - 1, 0);
        const int blk = __ldg(a.block_table + (int64_t)seq * a.bt_stride + pos / a.block_size);
        const bool ends_here = kv_end > kv_start && (r < rr.r_b || rr.rb_ends);
        if (ends_here && slot >= w.num_cache_slots) {
          if (c == 0 && w.err_flag) atomicOr(w.err_flag, TQ4_DEV_BAD_SLOT);
        } else if (ends_here && slot >= 0) {
          // the write is ordered before this call's reads only if the slot is the row's last position
          if ((int64_t)blk * a.block_size + pos % a.block_size != slot && c == 0 && w.err_flag)
            atomicOr(w.err_flag, TQ4_DEV_WRITE_ORDER);
          where = kRowWrite | (src ? kRowV : 0ull) |
                  (unsigned long long)(slot * w.cache_token_stride + (src ? lay.v_idx : lay.k_idx) + kvh * (D / 2));
        }
        src_ptr = src ? w.x[1] : w.x[0];
        src_dtype = w.x_dtype;
        ts = src ? w.token_stride[1] : w.token_stride[0];
        hs = src ? w.head_stride[1] : w.head_stride[0];
        base = (int64_t)tok * ts + (int64_t)kvh * hs;
      }
    }
    const int es = src_dtype == TQ4_F32 ? 4 : 2;
    const bool vec_ok = ((uintptr_t)src_ptr % 16 == 0) && (ts * es) % 16 == 0 && (hs * es) % 16 == 0;
    float x[R::KS][4];
#pragma unroll
    for (int s = 0; s < R::KS; ++s) {
      if (src_ptr) load_q4(src_ptr, src_dtype, base + 16 * s + 4 * c, vec_ok, x[s]);
      else x[s][0] = x[s][1] = x[s][2] = x[s][3] = 0.f;
    }
    // ---- squared norm in the order of the compress kernels: element k belongs to partial
    // l = k mod 32 (an ascending FMA chain over k = l, l + 32, ...), the partials are merged by the
    // butterfly 16, 8, 4, 2, 1.  This lane holds l = 4 c + e and l + 16 (k-steps 2 i and 2 i + 1).
    float pa[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float p0 = 0.f, p1 = 0.f;
#pragma unroll
      for (int i = 0; i < R::KS / 2; ++i) {
        p0 = fmaf(x[2 * i][e], x[2 * i][e], p0);
        p1 = fmaf(x[2 * i + 1][e], x[2 * i + 1][e], p1);
      }
      pa[e] = p0 + p1;                                                // l ^ 16
      pa[e] = pa[e] + __shfl_xor_sync(0xffffffffu, pa[e], 2);         // l ^ 8  (lane c ^ 2)
      pa[e] = pa[e] + __shfl_xor_sync(0xffffffffu, pa[e], 1);         // l ^ 4  (lane c ^ 1)
    }
    const float nrm = sqrtf((pa[0] + pa[2]) + (pa[1] + pa[3]));       // l ^ 2, l ^ 1
    // write vectors are normalised first (x * (1 / den) is within an ulp of x / den); then every
    // vector is scaled by the power of two that brings its largest element into [1, 2)
    const float pre = (where & kRowWrite) ? 1.f / (nrm + 1e-10f) : 1.f;
    float amax = 0.f;
#pragma unroll
    for (int s = 0; s < R::KS; ++s)
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        x[s][i] *= pre;
        amax = fmaxf(amax, fabsf(x[s][i]));
      }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    float sc = 1.f, isc = 1.f;
    if (amax > 0.f && amax < CUDART_INF_F) {
      const int exc = min(max((int)((__float_as_uint(amax) >> 23) & 0xFFu) - 127, -100), 100);
      sc = __uint_as_float((uint32_t)(127 - exc) << 23);
      isc = __uint_as_float((uint32_t)(127 + exc) << 23);
    }
#pragma unroll
    for (int s = 0; s < R::KS; ++s) {
      const float y[4] = {x[s][0] * sc, x[s][1] * sc, x[s][2] * sc, x[s][3] * sc};
      uint32_t h01, h23, l01, l23;
      split4(y, h01, h23, l01, l23);
      const uint32_t off = mem + rot_chunk_off<D>(row, 4 * s + c);
      asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(off), "r"(h01), "r"(h23) : "memory");
      asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(off + GroupMem<D>::kHalf), "r"(l01), "r"(l23) : "memory");
    }
    if (c == 0) {
      const uint32_t io = mem + GroupMem<D>::kInfo + row * 16;
      asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(io), "r"((uint32_t)where), "r"((uint32_t)(where >> 32)) : "memory");
      asm volatile("st.shared.v2.b32 [%0], {%1, %2};" ::"r"(io + 8), "r"(__float_as_uint(isc * (1.f / 256.f))),
                   "r"(__float_as_uint(nrm)) : "memory");
    }
  }
}

// One task: the 16 vectors of the group staged at `mem` times the output coordinates
// [16 nq, 16 nq + 16) of Pi (hi / lo fp16 at `tab`).
template <int D>
__device__ __forceinline__ void fused_mma_task(const AttnArgs& a, const CompressArgs& w, const float* s_bounds,
                                               uint32_t tab, uint32_t mem, int nq, int lane) {
  using R = RotCfg<D>;
  const int g = lane >> 2, c = lane & 3;
  // where the two vectors of this lane (g and g + 8) go
  unsigned long long where[2];
  float inv_scale[2], nrm[2];
#pragma unroll
  for (int hf = 0; hf < 2; ++hf) {
    uint32_t q4[4];
    lds_words<16>(mem + GroupMem<D>::kInfo + (g + 8 * hf) * 16, q4);
    where[hf] = (unsigned long long)q4[0] | ((unsigned long long)q4[1] << 32);
    inv_scale[hf] = __uint_as_float(q4[2]);
    nrm[hf] = __uint_as_float(q4[3]);
  }
  const bool any_row = !(where[0] & kRowInvalid) || !(where[1] & kRowInvalid);
  if (!__any_sync(0xffffffffu, any_row)) return;  // e.g. new tokens of rows that end in another CTA
  TQ4_STAMP(8);
  // 8-byte chunk 4 s + c of row n sits at n * PITCH + 8 * ((4 s + c) ^ x) with x = 4 * (n & 3) (no XOR
  // at head_dim 96); every row this lane touches (g, g + 8, 8 * block + g) has n & 3 = g & 3, so the
  // chunk offset of k-step s is the same for all of them
  const uint32_t gx = R::XOR ? (uint32_t)(g & 3) : 0u;
  const uint32_t a_row = mem + g * R::PITCH + 8 * c;
  // the n-blocks of the task advance together, each with a main (hi * hi) and a correction
  // (lo * hi + hi * lo) accumulator: independent chains of 8 / 16 dependent MMAs
  const uint32_t b_row = tab + (nq * 8 * R::NBT + g) * R::PITCH + 8 * c;
  float acc[R::NBT][4], cor[R::NBT][4];
#pragma unroll
  for (int j = 0; j < R::NBT; ++j)
#pragma unroll
    for (int e = 0; e < 4; ++e) acc[j][e] = cor[j][e] = 0.f;
#pragma unroll 2
  for (int s = 0; s < R::KS; ++s) {
    const uint32_t ko = 32u * ((uint32_t)s ^ gx);
    uint32_t ah0[2], ah1[2], al0[2], al1[2];
    lds_words<8>(a_row + ko, ah0);
    lds_words<8>(a_row + ko + 8 * R::PITCH, ah1);
    lds_words<8>(a_row + ko + GroupMem<D>::kHalf, al0);
    lds_words<8>(a_row + ko + GroupMem<D>::kHalf + 8 * R::PITCH, al1);
#pragma unroll
    for (int j = 0; j < R::NBT; ++j) {
      uint32_t bh[2], bl[2];
      lds_words<8>(b_row + ko + j * 8 * R::PITCH, bh);
      lds_words<8>(b_row + ko + j * 8 * R::PITCH + R::LO_BASE, bl);
      mma16816(acc[j], ah0[0], ah1[0], ah0[1], ah1[1], bh[0], bh[1]);
      mma16816(cor[j], al0[0], al1[0], al0[1], al1[1], bh[0], bh[1]);
      mma16816(cor[j], ah0[0], ah1[0], ah0[1], ah1[1], bl[0], bl[1]);
    }
  }
#pragma unroll 1
  for (int j = 0; j < R::NBT; ++j) {
    const int n0 = (nq * R::NBT + j) * 8 + 2 * c;  // C columns of this lane: coordinates n0 (even), n0 + 1
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      // (indexing the accumulators with the rolled j would spill them: select instead)
      float y0 = 0.f, y1 = 0.f;
#pragma unroll
      for (int jj = 0; jj < R::NBT; ++jj)
        if (jj == j) {
          y0 = (acc[jj][2 * hf] + cor[jj][2 * hf]) * inv_scale[hf];
          y1 = (acc[jj][2 * hf + 1] + cor[jj][2 * hf + 1]) * inv_scale[hf];
        }
      const unsigned long long wh = where[hf];
      if (wh & kRowInvalid) continue;
      if (!(wh & kRowWrite)) {
        *reinterpret_cast<float2*>(a.plan.q_rot + (int64_t)(wh & kRowOffMask) + n0) = make_float2(y0, y1);
      } else {
        const float* bd = s_bounds + ((wh & kRowV) ? 16 : 0);
        w.cache[(int64_t)(wh & kRowOffMask) + (n0 >> 1)] =
            (uint8_t)((bucketize_sorted16(y0, bd) << 4) | bucketize_sorted16(y1, bd));
      }
    }
  }
  // the fp32 norm of a written vector is stored once, by the task of the first 32 coordinates
  if (nq == 0 && c == 0) {
    const RowLayout lay = row_layout(a.sh.Hkv, D);
#pragma unroll
    for (int hf = 0; hf < 2; ++hf) {
      const unsigned long long wh = where[hf];
      if ((wh & kRowInvalid) || !(wh & kRowWrite)) continue;
      // index bytes of head h start at region + h * D/2, its norm at region_norm + h * 4
      const int64_t off = (int64_t)(wh & kRowOffMask);
      const int64_t row_start = off / w.cache_token_stride * w.cache_token_stride;
      const int in_row = (int)(off - row_start);
      const int region = (wh & kRowV) ? lay.v_idx : lay.k_idx;
      const int h = (in_row - region) / (D / 2);
      *reinterpret_cast<float*>(w.cache + row_start + ((wh & kRowV) ? lay.v_norm : lay.k_norm) + 4 * h) = nrm[hf];
    }
  }
  TQ4_STAMP(9);
}

// byte offset (within a head's D/2 V bytes) of this thread's m-block i
template <int D>
__device__ __forceinline__ int v_byte_of_mblock(int g, int i) {
  constexpr int VW = (D / 16) / 4;
  return i < 4 * VW ? g * 4 * VW + i : 32 * VW + 2 * g + (i - 4 * VW);
}

// BOX selects the TMA box scheme: 0 = four 3-D boxes per tile (K rows, V rows, K norms, V norms),
// 1 = the same with a 16-byte wider V box (V region not 16-byte aligned), 2 = two 4-D boxes per
// tile: the K and V halves of a token row have the same shape a fixed distance apart, so one box
// with an extra "half" dimension fetches both index tiles, and one both norm tiles.
template <int D, int NB, bool ALIGNED, bool PAGE16, int WARPS, bool TMA, int BOX>
__global__ void __launch_bounds__(WARPS * 32, 1)
attention_mma_kernel(const AttnArgs a, const CompressArgs w, const int has_write, const uint32_t smem_total,
                     const __grid_constant__ CUtensorMap tm_data,
                     const __grid_constant__ CUtensorMap tm_v,
                     const __grid_constant__ CUtensorMap tm_norm) {
  using C = MmaCfg<D, ALIGNED>;
  constexpr bool VWIDE = BOX == 1, MERGED = BOX == 2, ROWBOX = BOX == 3;
  constexpr bool V4B = VWIDE || ROWBOX;  // V chunks start on 4-byte (not 8/16-byte) boundaries
  constexpr int kRowPitch = (D + 8 + 15) & ~15;  // ROWBOX: one box holds the whole row of the only KV head
  constexpr int kTmaKN = C::template tma_kn<VWIDE>(), kTmaVN = kTmaKN + 256;
  constexpr int kTmaStage = ROWBOX ? 16 * kRowPitch : C::template tma_stage<VWIDE>();
  constexpr int kVPitch = ROWBOX ? kRowPitch : C::template v_pitch<VWIDE>();
  constexpr int kStage = TMA ? kTmaStage : C::kStageBytes;
  const AttnShape& sh = a.sh;
  const AttnPlan& p = a.plan;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  __shared__ float s_cent[2][TQ4_MAX_CENTROIDS];
  __shared__ __align__(8) uint64_t s_bar[WARPS][kStages];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;

  // ---- shared memory map: [rings A][64 KB table on a 64 KB boundary][rings B] ------------------
  const uint32_t base = smem_u32(smem_raw);
  const uint32_t tab = (base + (kTableBytes - 1)) & ~(kTableBytes - 1);
  constexpr uint32_t kRing = kStages * 2 * kStage;  // each ring stage holds a pair of tiles
  const uint32_t n_a = (tab - base) / kRing;
  const uint32_t end = base + smem_total;
  const uint32_t ring =
      warp < (int)n_a ? base + warp * kRing : tab + kTableBytes + (warp - n_a) * kRing;
  if (tab + kTableBytes > end || ring + kRing > end) {  // the host sized smem_total to fit
    pdl_wait();
    if (threadIdx.x == 0 && a.err_flag) atomicOr(a.err_flag, TQ4_DEV_TIMEOUT);
    return;
  }
  TQ4_STAMP(0);
  // ---- lane- and warp-constant addressing (pure arithmetic) ----------------------------------------
  const uint32_t lb_k = tab + lane * 4, lb_v = tab + 128 + lane * 4;
  const uint32_t bar0 = smem_u32(&s_bar[warp][0]);
  // Row g of the score MMA / k-slot of the PV MMA does not hold token g of the tile but token
  // sigma(g).  With the 64-byte TMA swizzle a tile row r starts in bank 16 * (r & 1) and its
  // 16-byte chunks are XORed with (r >> 1) & 3, so
  //  * the 16-byte K reads of a quarter warp (rows sigma(2p), sigma(2p+1), all four chunks) need
  //    two rows of different parity, and
  //  * the 8-byte V reads of a half warp (rows sigma(2c) or sigma(2c+1) for c = 0..3, chunks 0-1
  //    or 2-3) need four rows that differ in (bit 0, bit 2),
  // which this permutation provides: every shared-memory read of a tile is conflict-free.
  // (ROWBOX rows are 144 bytes apart and unswizzled: 0,2,4,6,1,3,5,7 keeps the 4-byte V reads at
  // the unavoidable two wavefronts and the 16-byte K reads at three per two)
  auto sigma = [](int k) {
    return (int)(((ROWBOX ? 0x75316420u : 0x65742130u) >> (4 * (k & 7))) & 7u) + (k & 8);  // 0,3,1,2,4,7,5,6
  };
  const int rg = sigma(g), rc0 = sigma(2 * c), rc1 = sigma(2 * c + 1);
  constexpr bool SWZ = TMA && D == 128 && !VWIDE && !ROWBOX;  // 64-byte rows: CU_TENSOR_MAP_SWIZZLE_64B
  const int cta = blockIdx.x % sh.ctas, slice = blockIdx.x / sh.ctas;
  const int vh = slice * sh.HPC + warp % sh.HPC, ts = warp / sh.HPC;
  const int kvh = vh / sh.NCH, chunk = vh % sh.NCH;
  const int qh0 = kvh * sh.G + chunk * sh.GC;
  const int gcount = min(sh.GC, sh.G - chunk * sh.GC);
  const RowLayout lay = row_layout(sh.Hkv, D);
  // byte offsets of this head's K norm / V indices / V norm relative to the 16-byte boundary below
  const int kn_sub = (lay.k_norm + 4 * kvh) & 15;
  const int vn_sub = (lay.v_norm + 4 * kvh) & 15;
  const int v_sub = VWIDE ? ((lay.v_idx + C::HALF * kvh) & 15) : 0;
  auto tile_off = [&](int row, int byte) -> uint32_t {  // offset of (row, byte) inside a [16][D/2] tile
    return SWZ ? (uint32_t)(row * 64 + ((((byte >> 4) ^ (row >> 1)) & 3) << 4) + (byte & 15))
               : (uint32_t)(row * C::HALF + byte);
  };
  // lane-constant byte offsets inside a TMA stage: K chunk of token sigma(g), V chunks of tokens
  // sigma(2c) / sigma(2c+1), norm columns of token sigma(g); tokens +8 are a fixed distance further
  // (ROWBOX: a stage row is the token row itself: [K idx D/2][K norm 4][V idx D/2][V norm 4])
  const uint32_t o_k = ROWBOX ? rg * kRowPitch + c * C::KBY : tile_off(rg, c * C::KBY);
  // (V bytes of a thread: 4 * VW bytes at g * 4 * VW, and at D = 96 a half-word at 32 * VW + 2 * g)
  constexpr int kVWordBytes = 4 * C::VW;
  const uint32_t o_v0 = ROWBOX ? rc0 * kRowPitch + C::HALF + 4 + g * kVWordBytes
                               : C::kTmaV + (VWIDE ? rc0 * kVPitch + v_sub + g * kVWordBytes : tile_off(rc0, g * kVWordBytes));
  const uint32_t o_v1 = ROWBOX ? rc1 * kRowPitch + C::HALF + 4 + g * kVWordBytes
                               : C::kTmaV + (VWIDE ? rc1 * kVPitch + v_sub + g * kVWordBytes : tile_off(rc1, g * kVWordBytes));
  const uint32_t o_vh0 = C::kTmaV + tile_off(rc0, 32 * C::VW + 2 * g);
  const uint32_t o_vh1 = C::kTmaV + tile_off(rc1, 32 * C::VW + 2 * g);
  const uint32_t o_kn = ROWBOX ? rg * kRowPitch + C::HALF : kTmaKN + rg * 16 + kn_sub;
  const uint32_t o_vn = ROWBOX ? rg * kRowPitch + D + 4 : kTmaKN + 256 + rg * 16 + vn_sub;
  constexpr uint32_t kRow8 = 8 * (ROWBOX ? kRowPitch : (SWZ ? 64 : C::HALF));
  constexpr uint32_t kVRow8 = 8 * (V4B ? kVPitch : (SWZ ? 64 : C::HALF));
  constexpr uint32_t kNormRow8 = ROWBOX ? 8 * kRowPitch : 128;
  uint32_t gk = 0;      // tiles this warp has pushed through the ring (stage = gk % kStages)
  bool dead = false;    // a bounded wait gave up: stop issuing work, fall through to the end
  // every warp phase streams its own contiguous span of the tile stream: span index = cta * TPC + ts
  const int span = cta * sh.TPC + ts;
  const int k_off = lay.k_idx + kvh * C::HALF + c * C::KBY;  // this thread's K chunk
  // x coordinates (bytes within a token row, 16-byte aligned) of this head's four TMA boxes
  const int x_k = lay.k_idx + kvh * C::HALF, x_v = (lay.v_idx + kvh * C::HALF) & ~15;
  const int x_kn = (lay.k_norm + kvh * 4) & ~15, x_vn = (lay.v_norm + kvh * 4) & ~15;
  const int kn_off = lay.k_norm + kvh * 4;
  const int vn_delta = lay.v_norm - lay.k_norm;              // V norm sits this far after the K norm
  const int v_off = lay.v_idx + kvh * C::HALF + g * 4 * C::VW;  // this thread's V word chunk
  const int vh_off = lay.v_idx + kvh * C::HALF + 32 * C::VW + 4 * (g >> 1);  // word with its half-word
  const uint32_t ts32 = (uint32_t)a.cache_token_stride;
  const int bs_shift = (a.block_size & (a.block_size - 1)) == 0 ? __ffs(a.block_size) - 1 : -1;

  // The box copies of one tile pair into ring stage st (tiles at positions pos and pos + 16 of pages
  // ba / bb; `two` = the second tile exists), issued by one elected lane onto the stage's barrier.
  // Returns the validity mask of the pair's 32 tokens (an out-of-range page is reported and masked).
  auto tma_issue_pair = [&](uint32_t st, int pos, int ba, int bb, bool two) -> uint32_t {
    const uint32_t nblk = (uint32_t)a.num_blocks;
    uint32_t okm = 0xFFFFFFFFu;
    if ((uint32_t)ba >= nblk || (two && (uint32_t)bb >= nblk)) {  // rare: report, mask the tile
      okm = ((uint32_t)ba < nblk ? 0xFFFFu : 0u) | ((uint32_t)bb < nblk ? 0xFFFF0000u : 0u);
      if (a.err_flag) atomicOr(a.err_flag, TQ4_DEV_BAD_BLOCK);
    }
    const uint32_t sb = ring + st * (2 * kStage), bar = bar0 + st * 8;
    const int bs_mask = a.block_size - 1;  // power of two (checked by the host)
    const int in_a = pos & bs_mask, in_b = (pos + kTileTokens) & bs_mask;
    if (elect_one()) {
      mbar_expect_tx(bar, two ? 2 * kTmaStage : kTmaStage);
      if (MERGED) {
        tma_load_4d(sb, &tm_data, x_k, in_a, 0, ba, bar);
        tma_load_4d(sb + kTmaKN, &tm_norm, x_kn, in_a, 0, ba, bar);
        if (two) {
          tma_load_4d(sb + kStage, &tm_data, x_k, in_b, 0, bb, bar);
          tma_load_4d(sb + kStage + kTmaKN, &tm_norm, x_kn, in_b, 0, bb, bar);
        }
      } else if (ROWBOX) {  // one box per tile: the 16 whole token rows of the only KV head
        tma_load_3d(sb, &tm_data, 0, in_a, ba, bar);
        if (two) tma_load_3d(sb + kStage, &tm_data, 0, in_b, bb, bar);
      } else {
        tma_load_3d(sb, &tm_data, x_k, in_a, ba, bar);
        tma_load_3d(sb + C::kTmaV, VWIDE ? &tm_v : &tm_data, x_v, in_a, ba, bar);
        tma_load_3d(sb + kTmaKN, &tm_norm, x_kn, in_a, ba, bar);
        tma_load_3d(sb + kTmaVN, &tm_norm, x_vn, in_a, ba, bar);
        if (two) {
          tma_load_3d(sb + kStage, &tm_data, x_k, in_b, bb, bar);
          tma_load_3d(sb + kStage + C::kTmaV, VWIDE ? &tm_v : &tm_data, x_v, in_b, bb, bar);
          tma_load_3d(sb + kStage + kTmaKN, &tm_norm, x_kn, in_b, bb, bar);
          tma_load_3d(sb + kStage + kTmaVN, &tm_norm, x_vn, in_b, bb, bar);
        }
      }
    }
    return okm;
  };

  // this warp's ring barriers (used by this warp only: warp-level ordering is enough)
  if (TMA && lane == 0) {
#pragma unroll
    for (int s = 0; s < kStages; ++s) mbar_init(smem_u32(&s_bar[warp][s]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  __syncwarp();

  // ---- plan state of the warp: its span and the row it is in ---------------------------------------
  int total = 0, tps = 1, t_begin = 0, t_end = 0;
  int r = 0;               // current row
  int f_t0 = 0, f_slot = 0;  // fused plan: first tile and first partial slot of row r
  bool pre_issued = false;   // fused plan: the first tile pair of the span is already in flight
  uint32_t pre_ok = 0xFFFFFFFFu;
  bool pre_can = false, pre_two = false;  // ... its position and page ids, fetched ahead of the issue
  int pre_pos = 0, pre_ba = 0, pre_bb = 0;

  // ---- fused prologue: tile plan, query rotation and the step's cache write ------------------------
  if (a.fused) {
    if constexpr (D <= 128) {
      const int n_warps = blockDim.x >> 5;
      const bool pi_one_batch = D * D / 4 <= kPiBatch * (int)blockDim.x;
      float4 pi_regs[kPiBatch];
      if (pi_one_batch) pi_load<D>(a.rotation, pi_regs);  // in flight while the plan is computed
      const WarpPlan wp = fused_plan(a, warp, n_warps, lane, span, cta * sh.TPC, sh.TPC);
      total = wp.total;
      tps = wp.tps;
      t_begin = (int)min((long long)span * tps, (long long)total);
      t_end = min(total, t_begin + tps);
      r = max(wp.r0, 0);
      f_t0 = wp.r0_t0;
      f_slot = wp.r0_slot;
      TQ4_STAMP(1);
      if constexpr (TMA) {
        // page ids of the span's first tile pair: fetched now, used after the rotation (the copies go
        // into the ring memory that stages the rotation's operands until then)
        if (t_begin < t_end && wp.r0 >= 0 && bs_shift >= 0) {
          int seq, kv_start, kv_end;
          decode_row_range(a, r, seq, kv_start, kv_end);
          const int seg_end = min(f_t0 + row_tiles(kv_start, kv_end), t_end);
          const int tile0 = kv_start / kTileTokens;
          const int last_pos = (tile0 + (seg_end - 1 - f_t0)) * kTileTokens;
          const int32_t* bt = a.block_table + (int64_t)seq * a.bt_stride;
          pre_pos = (tile0 + (t_begin - f_t0)) * kTileTokens;
          pre_two = pre_pos + kTileTokens <= last_pos;
          pre_ba = __ldg(bt + (pre_pos >> bs_shift));
          pre_bb = __ldg(bt + (min(pre_pos + kTileTokens, last_pos) >> bs_shift));
          pre_can = true;
        }
      }
      static_assert(GroupMem<D>::kBytes <= (int)kRing, "a group of 16 staged vectors fits a warp's ring memory");
      if (pi_one_batch) pi_store<D>(pi_regs, tab);
      else stage_rotation_split<D>(a.rotation, tab);
      if (has_write && threadIdx.x < 32) {  // sorted boundaries of K and V, padded with +inf
        const int src = threadIdx.x >> 4, i = threadIdx.x & 15;
        s_cent[src][i] = i < w.n_bounds[src] ? w.bounds[src][i] : CUDART_INF_F;
      }
      RotRows rr;
      rr.r_a = wp.r_a;
      rr.r_b = wp.r_b;
      rr.rb_ends = wp.rb_ends;
      {
        const int vh0 = slice * sh.HPC, vh1 = vh0 + sh.HPC - 1, c1 = vh1 % sh.NCH;
        rr.h0 = (vh0 / sh.NCH) * sh.G + (vh0 % sh.NCH) * sh.GC;
        rr.nh = (vh1 / sh.NCH) * sh.G + c1 * sh.GC + min(sh.GC, sh.G - c1 * sh.GC) - rr.h0;
        rr.kvh0 = vh0 / sh.NCH;
        rr.nkv = vh1 / sh.NCH - rr.kvh0 + 1;
      }
      const int n_rows = (wp.r_a >= 0 && wp.r_b >= wp.r_a) ? wp.r_b - wp.r_a + 1 : 0;
      rr.n_q = n_rows * rr.nh;
      rr.n_vec = rr.n_q + (has_write ? n_rows * 2 * rr.nkv : 0);
      const int n_groups = (rr.n_vec + 15) >> 4;
      auto ring_of = [&](int wi) -> uint32_t {
        return wi < (int)n_a ? base + wi * kRing : tab + kTableBytes + (wi - n_a) * kRing;
      };
#pragma unroll 1
      for (int g0 = 0; g0 == 0 || g0 < n_groups; g0 += n_warps) {  // (n_groups is the same in every warp of the CTA)
        if (g0 + warp < n_groups) fused_prep_group<D>(a, w, has_write != 0, rr, g0 + warp, ring, lane);
        __syncthreads();  // Pi and the round's groups are staged
        if (g0 == 0) TQ4_STAMP(2);
        const int n_round = min(n_warps, n_groups - g0);
#pragma unroll 1
        for (int t_ = warp; t_ < n_round * RotCfg<D>::NQ; t_ += n_warps)
          fused_mma_task<D>(a, w, &s_cent[0][0], tab, ring_of(t_ / RotCfg<D>::NQ), t_ % RotCfg<D>::NQ, lane);
        if (g0 + n_warps < n_groups) __syncthreads();  // the rings are staged again by the next round
      }
      TQ4_STAMP(10);
      // the written cache rows are read back by bulk tensor copies (async proxy) after the barrier
      if (has_write) asm volatile("fence.proxy.async.global;" ::: "memory");
      TQ4_STAMP(11);
    }
    __syncthreads();  // rotated queries and written tokens are visible to the block; the table region is free
    TQ4_STAMP(3);
    if constexpr (TMA) {
      // the first tile pair goes into flight now and lands while the table is built
      if (pre_can) {
        pre_ok = tma_issue_pair(0, pre_pos, pre_ba, pre_bb, pre_two);
        pre_issued = true;
      }
    }
  }
  // ---- replicated byte -> half2 tables: slot l < 32 = K table of lane l, slot 32 + l = V -------
  if (threadIdx.x < 2 * TQ4_MAX_CENTROIDS) {
    const int w_ = threadIdx.x >> 4, i = threadIdx.x & 15;
    const float* cent = w_ ? a.v_centroids : a.k_centroids;
    const int nc = w_ ? a.n_v_centroids : a.n_k_centroids;
    s_cent[w_][i] = i < nc ? __fmul_rn(w_ ? a.lut_scale_v : a.lut_scale_k, cent[i]) : 0.f;
  }
  __syncthreads();
  {
    // the 32 lane copies of an entry are contiguous: four per 16-byte store
    uint4* t = reinterpret_cast<uint4*>(smem_raw + (tab - base));
    for (int i = threadIdx.x; i < 256 * 16; i += blockDim.x) {
      const int byte = i >> 4, w_ = (i >> 3) & 1;
      const uint32_t v = pack_h2(s_cent[w_][byte >> 4], s_cent[w_][byte & 15]);
      t[i] = make_uint4(v, v, v, v);
    }
  }
  __syncthreads();
  // everything above used only caller inputs and shared memory (a launch with the fused prologue is
  // a plain one); without it the kernel now reads the plan and the rotated queries of the prologue
  // kernel and the cache the write kernel filled
  pdl_trigger();
  pdl_wait();
  TQ4_STAMP(4);
  if (!a.fused) {
    total = p.scalars[0];
    tps = p.scalars[1];
    t_begin = (int)min((long long)span * tps, (long long)total);
    t_end = min(total, t_begin + tps);
  }
  if (t_begin >= t_end) return;

  // first row of the span: the largest r with tile_prefix[r] <= t_begin (the array is
  // non-decreasing).  Two levels of 32-way search: two dependent memory round trips instead of
  // log2(rows) of a binary search.
  if (!a.fused) {
    const int rows = sh.rows;
    const int stride = (rows + 31) / 32;
    const int v1 = __ldg(p.tile_prefix + min(lane * stride, rows));
    const unsigned m1 = __ballot_sync(0xffffffffu, v1 <= t_begin);  // a prefix of the lanes (entry 0 is 0)
    const int base_i = (31 - __clz(m1 | 1u)) * stride;
    int best = base_i;
    for (int jj = lane; jj < stride; jj += 32) {
      const int i = base_i + jj;
      if (i < rows && __ldg(p.tile_prefix + i) <= t_begin) best = i;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) best = max(best, __shfl_xor_sync(0xffffffffu, best, o));
    r = min(best, rows - 1);
    while (p.tile_prefix[r + 1] <= t_begin) ++r;
  }

  int t = t_begin;
  while (t < t_end) {
    int row_t0, row_t1, kv_start, kv_end, row_seq;
    if (a.fused) {  // from the sequence length: the plan arrays are not read back
      decode_row_range(a, r, row_seq, kv_start, kv_end);
      row_t0 = f_t0;
      row_t1 = f_t0 + row_tiles(kv_start, kv_end);
    } else {
      row_t0 = p.tile_prefix[r];
      row_t1 = p.tile_prefix[r + 1];
      kv_start = p.kv_start[r];
      kv_end = p.kv_end[r];
      row_seq = p.row_seq[r];
    }
    const int seg_end = min(row_t1, t_end);
    const int32_t* bt = a.block_table + (int64_t)row_seq * a.bt_stride;
    const int tile0 = kv_start / kTileTokens;

    // ---- query fragments: column g of n-block nb = head nb*4 + g/2, term g%2 (hi / lo) ------
    uint32_t qf[NB][C::KS][2];
    float fscale[NB];  // qmax * sm_scale * log2(e) / alpha_k of head nb*4 + c
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      const int hh = nb * 4 + (g >> 1);
      float v[C::DPT];
      float qmax = 0.f;
      if (hh < gcount) {
        const float4* src = reinterpret_cast<const float4*>(
            p.q_rot + ((int64_t)r * sh.Hq + qh0 + hh) * D + c * C::DPT);
#pragma unroll
        for (int j = 0; j < C::DPT / 4; ++j) {
          const float4 x = src[j];
          v[4 * j] = x.x; v[4 * j + 1] = x.y; v[4 * j + 2] = x.z; v[4 * j + 3] = x.w;
        }
#pragma unroll
        for (int j = 0; j < C::DPT; ++j) qmax = fmaxf(qmax, fabsf(v[j]));
      } else {
#pragma unroll
        for (int j = 0; j < C::DPT; ++j) v[j] = 0.f;
      }
      qmax = fmaxf(qmax, __shfl_xor_sync(0xffffffffu, qmax, 1));
      qmax = fmaxf(qmax, __shfl_xor_sync(0xffffffffu, qmax, 2));
      const float inv = qmax > 0.f ? 1.f / qmax : 0.f;
      const bool lo_term = g & 1;
#pragma unroll
      for (int j = 0; j < C::DPT; ++j) {
        const float x = v[j] * inv;
        const float hi = __half2float(__float2half_rn(x));
        v[j] = lo_term ? x - hi : hi;
      }
#pragma unroll
      for (int s = 0; s < C::KS; ++s) {
        qf[nb][s][0] = pack_h2(v[4 * s], v[4 * s + 1]);
        qf[nb][s][1] = pack_h2(v[4 * s + 2], v[4 * s + 3]);
      }
      // head nb*4 + c lives in columns 2c, 2c+1: take its qmax from lane g' = 2c
      fscale[nb] = __shfl_sync(0xffffffffu, qmax, 8 * c) * (a.scale_log2e / a.lut_scale_k);
    }

    float m[NB], l[NB], acc[C::MB][NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      m[nb] = -CUDART_INF_F;
      l[nb] = 0.f;
#pragma unroll
      for (int i = 0; i < C::MB; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[i][nb][e] = 0.f;
    }

    auto pos0_of = [&](int tt) { return (tile0 + (tt - row_t0)) * kTileTokens; };
    auto page_of = [&](int pos0) { return bs_shift >= 0 ? (pos0 >> bs_shift) : (pos0 / a.block_size); };
    auto token_row = [&](int pos) -> const uint8_t* {  // generic addressing: one lookup per token
      const int pc = min(max(pos, kv_start), kv_end - 1);
      const int blk = __ldg(bt + pc / a.block_size);
      const bool ok = blk >= 0 && blk < a.num_blocks;
      return a.cache + (int64_t)(ok ? blk : 0) * a.cache_block_stride +
             (int64_t)(pc % a.block_size) * a.cache_token_stride;
    };
    // ---- issue the copies of one tile into ring stage st; returns 1 if its page is valid --------
    auto issue_tile = [&](int tt, int blk, uint32_t sb, uint32_t bar) -> uint32_t {
      const int pos0 = pos0_of(tt);
      uint32_t ok = 1;
      if (TMA) {  // the box copies themselves are issued by issue_pair under one election
        ok = blk >= 0 && blk < a.num_blocks;
        if (!ok && a.err_flag) atomicOr(a.err_flag, TQ4_DEV_BAD_BLOCK);
        return ok;
      }
      const uint8_t *rk0, *rk1, *rv[4];
      if (PAGE16) {
        ok = blk >= 0 && blk < a.num_blocks;
        if (!ok && a.err_flag) atomicOr(a.err_flag, TQ4_DEV_BAD_BLOCK);
        const int inpage = bs_shift >= 0 ? (pos0 & (a.block_size - 1)) : (pos0 % a.block_size);
        const uint8_t* pb = a.cache + (int64_t)(ok ? blk : 0) * a.cache_block_stride +
                            (int64_t)inpage * a.cache_token_stride;
        rk0 = pb + rg * ts32;
        rk1 = rk0 + 8 * ts32;
        rv[0] = pb + rc0 * ts32;
        rv[1] = pb + rc1 * ts32;
        rv[2] = rv[0] + 8 * ts32;
        rv[3] = rv[1] + 8 * ts32;
      } else {
        rk0 = token_row(pos0 + rg);
        rk1 = token_row(pos0 + rg + 8);
        rv[0] = token_row(pos0 + rc0);
        rv[1] = token_row(pos0 + rc1);
        rv[2] = token_row(pos0 + rc0 + 8);
        rv[3] = token_row(pos0 + rc1 + 8);
      }
#pragma unroll
      for (int u = 0; u < C::NK; ++u) {
        cp_async<C::UK>(sb + u * 32 * C::UK + lane * C::UK, rk0 + k_off + u * C::UK);
        cp_async<C::UK>(sb + C::kOffK1 + u * 32 * C::UK + lane * C::UK, rk1 + k_off + u * C::UK);
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint32_t vb = sb + C::kOffV + j * C::kVTok;
#pragma unroll
        for (int u = 0; u < C::NV; ++u)
          cp_async<C::UV>(vb + u * 32 * C::UV + lane * C::UV, rv[j] + v_off + u * C::UV);
        if (C::VH) cp_async<4>(vb + 32 * 4 * C::VW + lane * 4, rv[j] + vh_off);
      }
      const uint32_t nbase = sb + C::kOffN + lane * 16;
      cp_async<4>(nbase, rk0 + kn_off);
      cp_async<4>(nbase + 4, rk1 + kn_off);
      cp_async<4>(nbase + 8, rk0 + kn_off + vn_delta);
      cp_async<4>(nbase + 12, rk1 + kn_off + vn_delta);
      return ok;
    };
    // generic addressing only: validity of each of the tile's 16 tokens
    auto token_okmask = [&](int pos0) -> uint32_t {
      const int pos = min(max(pos0 + (lane & 15), kv_start), kv_end - 1);
      const int b = __ldg(bt + pos / a.block_size);
      const bool ok = b >= 0 && b < a.num_blocks;
      if (!ok && a.err_flag) atomicOr(a.err_flag, TQ4_DEV_BAD_BLOCK);
      return __ballot_sync(0xffffffffu, ok) & 0xFFFFu;
    };

    // ---- pieces of the per-tile work; sb = shared address of the tile's ring slot -----------------
    // K side of one tile: raw dots of (token g, head c) and (token g+8, head c) per n-block
    auto k_side = [&](uint32_t sb, float (&dots)[NB][2]) {
      uint32_t kw0[C::KW], kw1[C::KW];
      if (TMA) {
#pragma unroll
        for (int u = 0; u < C::NK; ++u) {
          // (a 16-byte chunk never straddles a swizzle unit: c * KBY + u * UK is a multiple of UK)
          lds_imm<C::UK, 0>(sb + o_k + u * C::UK, kw0 + u * (C::UK / 4));
          lds_imm<C::UK, kRow8>(sb + o_k + u * C::UK, kw1 + u * (C::UK / 4));
        }
      } else {
#pragma unroll
        for (int u = 0; u < C::NK; ++u) {
          lds_words<C::UK>(sb + u * 32 * C::UK + lane * C::UK, kw0 + u * (C::UK / 4));
          lds_words<C::UK>(sb + C::kOffK1 + u * 32 * C::UK + lane * C::UK, kw1 + u * (C::UK / 4));
        }
      }
      float sacc[NB][2][4];  // two independent accumulation chains per n-block
#pragma unroll
      for (int w = 0; w < C::KW; ++w) {
        const uint32_t w0 = kw0[w], w1 = kw1[w];
        {
          const uint32_t a0 = lut<0>(w0, lb_k), a2 = lut<1>(w0, lb_k);
          const uint32_t a1 = lut<0>(w1, lb_k), a3 = lut<1>(w1, lb_k);
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            if (w == 0) mma16816_zero(sacc[nb][0], a0, a1, a2, a3, qf[nb][0][0], qf[nb][0][1]);
            else mma16816(sacc[nb][0], a0, a1, a2, a3, qf[nb][2 * w][0], qf[nb][2 * w][1]);
          }
        }
        {
          const uint32_t a0 = lut<2>(w0, lb_k), a2 = lut<3>(w0, lb_k);
          const uint32_t a1 = lut<2>(w1, lb_k), a3 = lut<3>(w1, lb_k);
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            if (w == 0) mma16816_zero(sacc[nb][1], a0, a1, a2, a3, qf[nb][1][0], qf[nb][1][1]);
            else mma16816(sacc[nb][1], a0, a1, a2, a3, qf[nb][2 * w + 1][0], qf[nb][2 * w + 1][1]);
          }
        }
      }
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        dots[nb][0] = (sacc[nb][0][0] + sacc[nb][1][0]) + (sacc[nb][0][1] + sacc[nb][1][1]);
        dots[nb][1] = (sacc[nb][0][2] + sacc[nb][1][2]) + (sacc[nb][0][3] + sacc[nb][1][3]);
      }
    };
    auto load_norms = [&](uint32_t sb, float (&nrm)[4]) {  // kn(g), kn(g+8), vn(g), vn(g+8)
      if (TMA) {
        lds_imm<4, 0>(sb + o_kn, reinterpret_cast<uint32_t*>(nrm));
        lds_imm<4, kNormRow8>(sb + o_kn, reinterpret_cast<uint32_t*>(nrm + 1));
        if (V4B) {  // the two norm regions may sit at different offsets inside their 16-byte columns
          lds_imm<4, 0>(sb + o_vn, reinterpret_cast<uint32_t*>(nrm + 2));
          lds_imm<4, kNormRow8>(sb + o_vn, reinterpret_cast<uint32_t*>(nrm + 3));
        } else {
          lds_imm<4, 256>(sb + o_kn, reinterpret_cast<uint32_t*>(nrm + 2));
          lds_imm<4, 384>(sb + o_kn, reinterpret_cast<uint32_t*>(nrm + 3));
        }
      } else {
        lds_words<16>(sb + C::kOffN + lane * 16, reinterpret_cast<uint32_t*>(nrm));
      }
    };
    // V side of one tile: O^T += V^T * Psplit^T with the tile's probability fragments
    auto v_side = [&](uint32_t sb, const uint32_t (&pf)[NB][2]) {
      uint32_t vw[4][C::VW + C::VH];  // tokens 2c, 2c+1, 2c+8, 2c+9
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (TMA) {
          const uint32_t vo = sb + ((j & 1) ? o_v1 : o_v0);
          if (V4B) {  // 4-byte reads: the chunk may start on any 4-byte boundary
#pragma unroll
            for (int u = 0; u < C::VW; ++u) {
              if (j < 2) lds_imm<4, 0>(vo + 4 * u, vw[j] + u);
              else lds_imm<4, kVRow8>(vo + 4 * u, vw[j] + u);
            }
          } else {
#pragma unroll
            for (int u = 0; u < C::NV; ++u) {
              if (j < 2) lds_imm<C::UV, 0>(vo + u * C::UV, vw[j] + u * (C::UV / 4));
              else lds_imm<C::UV, kVRow8>(vo + u * C::UV, vw[j] + u * (C::UV / 4));
            }
            if (C::VH) {  // D = 96: the thread's last two V bytes, in the low half of the word
              const uint32_t ho = sb + ((j & 1) ? o_vh1 : o_vh0) + (j < 2 ? 0u : kVRow8);
              asm volatile("ld.shared.u16 %0, [%1];" : "=r"(vw[j][C::VW]) : "r"(ho));
            }
          }
        } else {
          const uint32_t vb = sb + C::kOffV + j * C::kVTok;
#pragma unroll
          for (int u = 0; u < C::NV; ++u)
            lds_words<C::UV>(vb + u * 32 * C::UV + lane * C::UV, vw[j] + u * (C::UV / 4));
          if (C::VH) {
            uint32_t x;
            lds_words<4>(vb + 32 * 4 * C::VW + lane * 4, &x);
            vw[j][C::VW] = (g & 1) ? (x >> 16) : (x & 0xFFFFu);
          }
        }
      }
#pragma unroll
      for (int w = 0; w < C::VW + C::VH; ++w) {
        const uint32_t x0 = vw[0][w], y0 = vw[1][w], x1 = vw[2][w], y1 = vw[3][w];
        const uint32_t ee0 = (x0 & 0xF0F0F0F0u) | ((y0 >> 4) & 0x0F0F0F0Fu);
        const uint32_t oo0 = ((x0 << 4) & 0xF0F0F0F0u) | (y0 & 0x0F0F0F0Fu);
        const uint32_t ee1 = (x1 & 0xF0F0F0F0u) | ((y1 >> 4) & 0x0F0F0F0Fu);
        const uint32_t oo1 = ((x1 << 4) & 0xF0F0F0F0u) | (y1 & 0x0F0F0F0Fu);
        const int i0 = 4 * w;
#define TQ4_V_STEP(J)                                                                          \
  if (i0 + J < C::MB) {                                                                        \
    const uint32_t a0 = lut<J>(ee0, lb_v), a1 = lut<J>(oo0, lb_v);                              \
    const uint32_t a2 = lut<J>(ee1, lb_v), a3 = lut<J>(oo1, lb_v);                              \
    _Pragma("unroll") for (int nb = 0; nb < NB; ++nb)                                          \
        mma16816(acc[i0 + J][nb], a0, a1, a2, a3, pf[nb][0], pf[nb][1]);                       \
  }
        TQ4_V_STEP(0)
        TQ4_V_STEP(1)
        TQ4_V_STEP(2)
        TQ4_V_STEP(3)
#undef TQ4_V_STEP
      }
    };

    // ---- one pair of consecutive tiles (32 tokens) from ring stage st -----------------------------
    // okmask: bits 0-15 tile A, bits 16-31 tile B; has2 = tile B exists
    // A missing tile B (odd tail of a segment) is still run through the arithmetic on whatever its
    // ring slot holds: every byte decodes to a finite centroid, and its tokens are masked below.
    auto compute_pair = [&](int st, int pos0, uint32_t okmask, bool has2) {
      const uint32_t sbA = ring + st * (2 * kStage), sbB = sbA + kStage;
      float dots[2][NB][2];
      float nrm[2][4];
      k_side(sbA, dots[0]);
      load_norms(sbA, nrm[0]);
      k_side(sbB, dots[1]);
      load_norms(sbB, nrm[1]);
      // token slots of this lane: (tile u, half h) = position pos0 + 16u + sigma(g) + 8h
      float kn[2][2], vn[2][2], lg[2][2], bias[2][2];
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          kn[u][h] = nrm[u][h];
          vn[u][h] = nrm[u][2 + h];
          bias[u][h] = 0.f;
        }
      const bool full = has2 && pos0 >= kv_start && pos0 + 2 * kTileTokens <= kv_end &&
                        okmask == 0xFFFFFFFFu;
      if (!full) {  // first / last tiles of a row, missing second tile, bad page: per-token masks
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int pp = pos0 + 16 * u + rg + 8 * h;
            const bool ok = (u == 0 || has2) && pp >= kv_start && pp < kv_end &&
                            ((okmask >> (16 * u + rg + 8 * h)) & 1u);
            if (!ok) { vn[u][h] = 0.f; kn[u][h] = 0.f; bias[u][h] = -CUDART_INF_F; }
          }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int h = 0; h < 2; ++h) lg[u][h] = fmaxf(lg2_approx(vn[u][h]), -30.f);
      // Online softmax with a lazily updated reference: m only moves when some score (shifted by
      // log2 of its value norm) exceeds it by more than 2^8, so the cross-lane max reduction and
      // the accumulator rescale run a handful of times per row; probabilities stay below 2^8.
      float s[NB][2][2];
      bool need = false;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            s[nb][u][h] = fmaf(dots[u][nb][h], fscale[nb] * kn[u][h], bias[u][h]);  // masked: -inf
            need |= s[nb][u][h] + lg[u][h] > m[nb] + 8.f;
          }
      if (__any_sync(0xffffffffu, need)) {
        asm volatile("" ::: "memory");  // rare path: keep it a real branch
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          float mt = fmaxf(fmaxf(s[nb][0][0] + lg[0][0], s[nb][0][1] + lg[0][1]),
                           fmaxf(s[nb][1][0] + lg[1][0], s[nb][1][1] + lg[1][1]));
          mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 4));
          mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 8));
          mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 16));
          if (mt > m[nb] + 8.f) {  // uniform over the 8 lanes that share head c
            const float alpha = m[nb] == -CUDART_INF_F ? 0.f : ex2_approx(m[nb] - mt);
            m[nb] = mt;
            l[nb] *= alpha;
#pragma unroll
            for (int i = 0; i < C::MB; ++i)
#pragma unroll
              for (int e = 0; e < 4; ++e)
                asm volatile("mul.f32 %0, %0, %1;" : "+f"(acc[i][nb][e]) : "f"(alpha));
          }
        }
      }
      uint32_t pf[2][NB][2];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        const float m_use = m[nb] == -CUDART_INF_F ? 0.f : m[nb];
        float lsum = 0.f;
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const float e = ex2_approx(s[nb][u][h] - m_use);
            lsum += e;
            pf[u][nb][h] = movmatrix_trans(split_h2(e * vn[u][h]));
          }
        l[nb] += lsum;
      }
      v_side(sbA, pf[0]);
      v_side(sbB, pf[1]);
    };

    // ---- stream the segment (TMA): two ring stages of one tile pair each ---------------------------
    // Steady state per pair: one election issuing the next pair's boxes, two block-table reads
    // for the pair after that, one bounded barrier wait, the arithmetic.  Positions advance by
    // additions; block-table reads past the segment are clamped to its last tile (never issued).
    if constexpr (TMA) {
      static_assert(kStages == 2, "the TMA loop alternates between two stages");
      const int step = 2;
      const int first = t;
      const int n_pairs = (first < seg_end && !dead) ? (seg_end - first + step - 1) / step : 0;
      if (n_pairs > 0) {
        const int step_tok = step * kTileTokens;
        const int last_pos = pos0_of(seg_end - 1);  // first token of the segment's last tile
        auto load_blk = [&](int pos) -> int { return __ldg(bt + (min(pos, last_pos) >> bs_shift)); };
        auto issue = [&](uint32_t st, int pos, int ba, int bb) -> uint32_t {
          return tma_issue_pair(st, pos, ba, bb, pos + kTileTokens <= last_pos);
        };
        uint32_t st = gk & 1u, ph = (gk >> 1) & 1u;  // stage and barrier parity of the current pair
        int pos_i = pos0_of(first), pos_c = pos_i;
        int blk_a = load_blk(pos_i), blk_b = load_blk(pos_i + kTileTokens);
        __syncwarp();
        uint32_t ok_cur = pre_issued ? pre_ok : issue(st, pos_i, blk_a, blk_b);  // (pre-issued: stage 0, gk == 0)
        pre_issued = false;
        pos_i += step_tok;
        blk_a = load_blk(pos_i);
        blk_b = load_blk(pos_i + kTileTokens);
        for (int k = 0; k < n_pairs; ++k) {
          __syncwarp();  // every lane has finished reading the stage about to be refilled
          uint32_t ok_next = 0xFFFFFFFFu;
          if (k + 1 < n_pairs) {
            ok_next = issue(st ^ 1u, pos_i, blk_a, blk_b);
            pos_i += step_tok;
            blk_a = load_blk(pos_i);
            blk_b = load_blk(pos_i + kTileTokens);
          }
          if (!mbar_wait_bounded(bar0 + st * 8, ph)) {
            if (lane == 0 && a.err_flag) atomicOr(a.err_flag, TQ4_DEV_TIMEOUT);
            dead = true;
            break;
          }
          if (gk == 0 && k == 0) TQ4_STAMP(5);
          compute_pair(st, pos_c, ok_cur, pos_c + kTileTokens <= last_pos);
          pos_c += step_tok;
          ok_cur = ok_next;
          ph ^= st;
          st ^= 1u;
        }
        gk += n_pairs;
      }
    } else
    // ---- stream the segment: kStages ring stages of one tile pair each; block ids one pair ahead ----
    {
      const int step = 2;
      const int first = t;
      const int n_pairs = (first < seg_end && !dead) ? (seg_end - first + step - 1) / step : 0;
      auto blk_of = [&](int tt) -> int { return (PAGE16 && tt < seg_end) ? __ldg(bt + page_of(pos0_of(tt))) : 0; };
      // issue both tiles of pair index pi into its ring stage; returns the pair's 2 validity bits
      auto issue_pair = [&](int pi, int blk_a, int blk_b, uint32_t use) -> uint32_t {
        const int ta = first + pi * step;
        const bool two = ta + 1 < seg_end;
        const uint32_t sb = ring + (use % kStages) * (2 * kStage);
        const uint32_t bar = bar0 + (use % kStages) * 8;
        uint32_t okb = issue_tile(ta, blk_a, sb, bar);
        if (two) okb |= issue_tile(ta + 1, blk_b, sb + kStage, bar) << 1;
        if (TMA) {
          // four box copies per tile by one elected lane: K rows, V rows, K-norm and V-norm columns
          const int pos_a = pos0_of(ta);
          const int in_a = bs_shift >= 0 ? (pos_a & (a.block_size - 1)) : (pos_a % a.block_size);
          const int in_b = bs_shift >= 0 ? ((pos_a + kTileTokens) & (a.block_size - 1))
                                         : ((pos_a + kTileTokens) % a.block_size);
          if (elect_one()) {
            mbar_expect_tx(bar, two ? 2 * kTmaStage : kTmaStage);
            tma_load_3d(sb, &tm_data, x_k, in_a, blk_a, bar);
            tma_load_3d(sb + C::kTmaV, VWIDE ? &tm_v : &tm_data, x_v, in_a, blk_a, bar);
            tma_load_3d(sb + kTmaKN, &tm_norm, x_kn, in_a, blk_a, bar);
            tma_load_3d(sb + kTmaVN, &tm_norm, x_vn, in_a, blk_a, bar);
            if (two) {
              tma_load_3d(sb + kStage, &tm_data, x_k, in_b, blk_b, bar);
              tma_load_3d(sb + kStage + C::kTmaV, VWIDE ? &tm_v : &tm_data, x_v, in_b, blk_b, bar);
              tma_load_3d(sb + kStage + kTmaKN, &tm_norm, x_kn, in_b, blk_b, bar);
              tma_load_3d(sb + kStage + kTmaVN, &tm_norm, x_vn, in_b, blk_b, bar);
            }
          }
        }
        if (!TMA) cp_async_commit();
        return okb;
      };
      if (n_pairs > 0) {
        uint32_t okbits = 0;  // 2 bits per in-flight pair, oldest first
#pragma unroll
        for (int s = 0; s < kStages - 1; ++s) {
          if (s < n_pairs)
            okbits |= issue_pair(s, blk_of(first + s * step), blk_of(first + s * step + 1), gk + s) << (2 * s);
          else if (!TMA)
            cp_async_commit();
        }
        int blk_a = blk_of(first + (kStages - 1) * step), blk_b = blk_of(first + (kStages - 1) * step + 1);
        for (int k = 0; k < n_pairs; ++k) {
          const int kn = k + kStages - 1;
          if (TMA) __syncwarp();  // every lane has finished reading the stage about to be refilled
          if (kn < n_pairs)
            okbits |= issue_pair(kn, blk_a, blk_b, gk + kn) << (2 * (kStages - 1));
          else if (!TMA)
            cp_async_commit();
          if (kn + 1 < n_pairs) {
            blk_a = blk_of(first + (kn + 1) * step);
            blk_b = blk_of(first + (kn + 1) * step + 1);
          }
          const int ta = first + k * step;
          const bool has2 = ta + 1 < seg_end;
          const int pos0 = pos0_of(ta);
          uint32_t okmask;
          if (PAGE16) {
            okmask = ((okbits & 1u) ? 0xFFFFu : 0u) | ((okbits & 2u) ? 0xFFFF0000u : 0u);
          } else {
            okmask = token_okmask(pos0);
            if (has2) okmask |= token_okmask(pos0 + kTileTokens) << 16;
          }
          okbits >>= 2;
          const uint32_t use = gk + k;
          if (TMA) {
            if (!mbar_wait_bounded(bar0 + (use % kStages) * 8, (use / kStages) & 1u)) {
              if (lane == 0 && a.err_flag) atomicOr(a.err_flag, TQ4_DEV_TIMEOUT);
              dead = true;
              break;
            }
          } else {
            cp_async_wait<kStages - 1>();
          }
          compute_pair(use % kStages, pos0, okmask, has2);
        }
        if (!TMA) cp_async_wait<0>();
        gk += n_pairs;
      }
    }

    TQ4_STAMP(6);
    // ---- write this warp's partial for the segment ---------------------------------------------
    const int slot = (a.fused ? f_slot : p.slot_base[r]) + (span - row_t0 / tps);
    const int64_t pidx = slot;
    const float inv_av = 1.f / a.lut_scale_v;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      float ls = l[nb];
      ls += __shfl_xor_sync(0xffffffffu, ls, 4);
      ls += __shfl_xor_sync(0xffffffffu, ls, 8);
      ls += __shfl_xor_sync(0xffffffffu, ls, 16);
      const int hh = nb * 4 + c;
      if (hh < gcount) {
        const int64_t hidx = pidx * sh.Hq + qh0 + hh;
        if (g == 0) {
          p.part_m[hidx] = dead ? -CUDART_INF_F : m[nb];
          p.part_l[hidx] = dead ? 0.f : ls;
        }
        float* dst = p.part_o + hidx * D;
#pragma unroll
        for (int i = 0; i < C::MB; ++i) {
          const int vb = v_byte_of_mblock<D>(g, i);
          *reinterpret_cast<float2*>(dst + 2 * vb) = make_float2(
              (acc[i][nb][0] + acc[i][nb][1]) * inv_av, (acc[i][nb][2] + acc[i][nb][3]) * inv_av);
        }
      }
    }
    t = seg_end;
    if (t < t_end) {
      if (a.fused) {  // next row that has tiles; its first tile and first partial slot follow from this row's
        f_slot += (row_t1 - 1) / tps - row_t0 / tps + 1;
        f_t0 = row_t1;
        for (++r; r < sh.rows - 1; ++r) {
          int sq, st_, en_;
          decode_row_range(a, r, sq, st_, en_);
          if (en_ > st_) break;
        }
      } else {
        ++r;
        while (p.tile_prefix[r + 1] <= t) ++r;
      }
    }
  }
  TQ4_STAMP(7);
}

// ---- TMA tensor maps over the paged cache: dims (row bytes, tokens in a block, blocks) -----------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

bool make_cache_map(CUtensorMap* m, const AttnArgs& a, uint32_t box_bytes, bool swizzle64) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t dims[3] = {(cuuint64_t)a.cache_token_stride, (cuuint64_t)a.block_size,
                              (cuuint64_t)a.num_blocks};
  const cuuint64_t strides[2] = {(cuuint64_t)a.cache_token_stride, (cuuint64_t)a.cache_block_stride};
  const cuuint32_t box[3] = {box_bytes, (cuuint32_t)kTileTokens, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(a.cache), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// 4-D map over the paged cache: dims (bytes of one half of a token row, tokens in a block, half, blocks).
// The K half [K indices | K norms] and the V half of a row have the same shape, H * (D/2 + 4) bytes apart.
bool make_cache_map_halves(CUtensorMap* m, const AttnArgs& a, uint32_t box_bytes, bool swizzle64) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return false;
  const cuuint64_t half_bytes = (cuuint64_t)a.sh.Hkv * (a.sh.D / 2 + 4);
  const cuuint64_t dims[4] = {half_bytes, (cuuint64_t)a.block_size, 2, (cuuint64_t)a.num_blocks};
  const cuuint64_t strides[3] = {(cuuint64_t)a.cache_token_stride, half_bytes, (cuuint64_t)a.cache_block_stride};
  const cuuint32_t box[4] = {box_bytes, (cuuint32_t)kTileTokens, 2, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 4, const_cast<uint8_t*>(a.cache), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_NONE,
            CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

constexpr int kErrNoHalvesMap = -1000;  // internal: the 4-D map could not be encoded, use 3-D boxes

template <int D, int NB, bool ALIGNED, bool PAGE16, bool TMA, int BOX>
int launch_mma_t(const AttnArgs& a, cudaStream_t st) {
  constexpr bool VWIDE = BOX == 1;
  constexpr int kRowPitch = (D + 8 + 15) & ~15;
  constexpr int WARPS = (D * NB <= 128) ? 16 : 8;  // upper bound; the launch uses HPC * TPC warps
  using C = MmaCfg<D, ALIGNED>;
  // All opt-in shared memory of the SM (one CTA per SM by design): the 64 KB table sits on a
  // 64 KB boundary of the shared window and whole rings are packed on both sides of it.
  constexpr auto kern = attention_mma_kernel<D, NB, ALIGNED, PAGE16, WARPS, TMA, BOX>;
  static int smem_avail[kMaxDevices];  // opt-in limit minus the kernel's static shared memory, per device
  const int dev = device_ordinal();
  if (dev < 0) return TQ4_ERR_CUDA;
  if (smem_avail[dev] == 0) {
    int optin = 0;
    cudaDeviceGetAttribute(&optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    cudaFuncAttributes fa;
    if (cudaFuncGetAttributes(&fa, kern) != cudaSuccess) return TQ4_ERR_CUDA;
    smem_avail[dev] = optin - (int)fa.sharedSizeBytes;  // static + dynamic share the opt-in limit
  }
  const int smem_total = smem_avail[dev];
  const int stage = TMA ? (BOX == 3 ? 16 * kRowPitch : C::template tma_stage<VWIDE>()) : C::kStageBytes;
  // the table may have to move up by almost its own size to reach a 64 KB boundary
  if (smem_total < (int)kTableBytes + a.sh.HPC * a.sh.TPC * kStages * 2 * stage) return TQ4_ERR_UNSUPPORTED;
  if (!ensure_dynamic_smem<kern>(smem_total)) return TQ4_ERR_CUDA;
  CUtensorMap tm_data, tm_v, tm_norm;
  memset(&tm_data, 0, sizeof(tm_data));
  memset(&tm_v, 0, sizeof(tm_v));
  memset(&tm_norm, 0, sizeof(tm_norm));
  if (TMA && BOX == 3) {
    if (!make_cache_map(&tm_data, a, kRowPitch, false)) return TQ4_ERR_CUDA;
  } else if (TMA && BOX == 2) {
    if (!make_cache_map_halves(&tm_data, a, D / 2, D == 128) || !make_cache_map_halves(&tm_norm, a, 16, false))
      return kErrNoHalvesMap;
  } else if (TMA && (!make_cache_map(&tm_data, a, D / 2, D == 128 && !VWIDE) ||
                     !make_cache_map(&tm_v, a, D / 2 + 16, false) || !make_cache_map(&tm_norm, a, 16, false))) {
    return TQ4_ERR_CUDA;
  }
  const int warps = a.sh.HPC * a.sh.TPC;
  static const CompressArgs no_write{};
  // with the fused prologue this is the first kernel to read the caller's tensors: a plain launch
  if (launch_kernel(kern, dim3(a.sh.ctas * a.sh.n_slices), dim3(warps * 32), (size_t)smem_total, st, !a.fused, a,
                    a.fused && a.fused_write ? *a.fused_write : no_write, a.fused && a.fused_write ? 1 : 0,
                    (uint32_t)smem_total, tm_data, tm_v, tm_norm) != cudaSuccess)
    return TQ4_ERR_CUDA;
  TQ4_CHECK_LAUNCH();
  return TQ4_OK;
}

bool cache_aligned(const AttnShape& sh, const uint8_t* cache, int64_t bs, int64_t ts) {
  // 16-byte K chunks and 8/16-byte V chunks need the regions of a token row aligned accordingly
  const RowLayout lay = row_layout(sh.Hkv, sh.D);
  const int valign = sh.D >= 256 ? 16 : 8;
  return ((uintptr_t)cache % 16 == 0) && bs % 16 == 0 && ts % 16 == 0 && lay.v_idx % valign == 0 &&
         (sh.D / 2) % valign == 0 && sh.D != 96;
}

// TMA boxes start on 16-byte boundaries of the token row: every region offset of every head must
// be a multiple of 16 (true whenever the number of KV heads is a multiple of 4).
// V indices of a head start on a 16-byte boundary of the row (true when Hkv is a multiple of 4);
// otherwise the V box is fetched 16 bytes wider from the boundary below (VWIDE).
bool cache_tma_ok(const AttnArgs& a) {
  return (uintptr_t)a.cache % 16 == 0 && a.cache_block_stride % 16 == 0 && a.cache_token_stride % 16 == 0 &&
         a.block_size % kTileTokens == 0 && a.block_size <= 256 &&
         (a.block_size & (a.block_size - 1)) == 0 && (a.sh.D / 2) % 16 == 0 &&
         a.cache_token_stride >= (int64_t)((row_data_bytes(a.sh.Hkv, a.sh.D) + 15) & ~15) &&
         a.num_blocks < (1ll << 31) && getenv("TQ4_NO_TMA") == nullptr && encode_tiled_fn() != nullptr;
}
// a single KV head (e.g. one rank of an 8-way head-sharded Llama): the whole token row fits one box
bool rowbox_ok(int Hkv, int D, int64_t token_stride) {
  return Hkv == 1 && (D == 64 || D == 128) && token_stride >= ((D + 8 + 15) & ~15);
}
bool cache_v_aligned16(const AttnArgs& a) {
  const RowLayout lay = row_layout(a.sh.Hkv, a.sh.D);
  return lay.v_idx % 16 == 0;
}

template <int D, int NB>
int launch_mma_dn(const AttnArgs& a, cudaStream_t st) {
  const bool aligned = cache_aligned(a.sh, a.cache, a.cache_block_stride, a.cache_token_stride);
  const bool page16 = a.block_size % kTileTokens == 0;
  if constexpr (D == 96) {
    // 48-byte index rows: the halves boxes work as for the other head dims; shared-memory reads
    // are 4-byte words plus a half-word (the unaligned unit sizes)
    if (cache_tma_ok(a) && cache_v_aligned16(a)) {
      static bool halves_ok96 = true;
      if (halves_ok96) {
        const int rc = launch_mma_t<D, NB, false, true, true, 2>(a, st);
        if (rc != kErrNoHalvesMap) return rc;
        halves_ok96 = false;
      }
    }
  }
  if (D != 96 && cache_tma_ok(a)) {
    if (cache_v_aligned16(a)) {
      static bool halves_ok = true;  // cleared if the driver refuses the 4-D map
      if (halves_ok) {
        const int rc = launch_mma_t<D, NB, true, true, (D != 96), (D != 96) ? 2 : 0>(a, st);
        if (rc != kErrNoHalvesMap) return rc;
        halves_ok = false;
      }
      return launch_mma_t<D, NB, true, true, (D != 96), 0>(a, st);
    }
    if (rowbox_ok(a.sh.Hkv, D, a.cache_token_stride))
      return launch_mma_t<D, NB, true, true, (D != 96), (D == 64 || D == 128) ? 3 : 0>(a, st);
    return launch_mma_t<D, NB, true, true, (D != 96), (D != 96) ? 1 : 0>(a, st);
  }
  if (aligned && page16) return launch_mma_t<D, NB, true, true, false, false>(a, st);
  if (aligned) return launch_mma_t<D, NB, true, false, false, false>(a, st);
  if (page16) return launch_mma_t<D, NB, false, true, false, false>(a, st);
  return launch_mma_t<D, NB, false, false, false, false>(a, st);
}

template <int D>
int launch_mma_d(const AttnArgs& a, cudaStream_t st) {
  return a.sh.GC <= 4 ? launch_mma_dn<D, 1>(a, st) : launch_mma_dn<D, 2>(a, st);
}

}  // namespace

int mma_warps_per_cta(int D, int GC, int Hkv, int64_t token_stride) {
  if (D * (GC <= 4 ? 1 : 2) > 128) return 8;
  if (rowbox_ok(Hkv, D, token_stride)) return 16;
  return Hkv % 4 == 0 ? 16 : 12;  // wider V tiles need more ring space per warp
}

bool attention_mma_supported(const AttnShape& sh, int block_size, const uint8_t* cache,
                             int64_t block_stride, int64_t token_stride) {
  (void)block_size; (void)cache; (void)block_stride;
  return supported_head_dim(sh.D) && sh.GC <= 8 && token_stride % 4 == 0;
}

#ifdef TQ4_TRACE
}  // namespace tq4
// Copies the 160 x 16 x 16 timeline stamps of the last launch to the host (tuning builds only).
extern "C" int tq4_trace_read(long long* out) {
  return cudaMemcpyFromSymbol(out, tq4::g_trace, sizeof(long long) * 160 * 16 * 16) == cudaSuccess ? 0 : 1;
}
namespace tq4 {
#endif

int launch_attention_mma(const AttnArgs& a, cudaStream_t st) {
  switch (a.sh.D) {
    case 64: return launch_mma_d<64>(a, st);
    case 96: return launch_mma_d<96>(a, st);
    case 128: return launch_mma_d<128>(a, st);
    case 256: return launch_mma_d<256>(a, st);
  }
  return TQ4_ERR_UNSUPPORTED;
}

}  // namespace tq4
