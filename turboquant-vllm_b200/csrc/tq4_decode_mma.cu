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
// knorm in fp32, probabilities by vnorm before the split.  Packed bytes go global -> registers
// directly (each byte is used once); the next tile is prefetched while the current one is
// consumed.
#include <math_constants.h>

#include "tq4_attention.cuh"

namespace tq4 {

namespace {

constexpr uint32_t kTableBytes = 65536;
constexpr uint32_t kMmaSmemBytes = 2 * kTableBytes;  // slack to reach a 64 KB boundary

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

__device__ __forceinline__ uint32_t ldg_stream_b32(const uint8_t* p) {
  uint32_t v;
  asm volatile("ld.global.nc.L1::no_allocate.b32 %0, [%1];" : "=r"(v) : "l"(p));
  return v;
}
__device__ __forceinline__ uint32_t ldg_stream_b16(const uint8_t* p) {
  uint16_t v;
  asm volatile("ld.global.nc.L1::no_allocate.b16 %0, [%1];" : "=h"(v) : "l"(p));
  return (uint32_t)v;
}
__device__ __forceinline__ void ldg_stream_v2(const uint8_t* p, uint32_t& a, uint32_t& b) {
  asm volatile("ld.global.nc.L1::no_allocate.v2.b32 {%0,%1}, [%2];" : "=r"(a), "=r"(b) : "l"(p));
}
__device__ __forceinline__ void ldg_stream_v4(const uint8_t* p, uint32_t& a, uint32_t& b,
                                              uint32_t& c, uint32_t& d) {
  asm volatile("ld.global.nc.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(a), "=r"(b), "=r"(c), "=r"(d)
               : "l"(p));
}
__device__ __forceinline__ float ldg_f32(const uint8_t* p) {
  float v;
  asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
  return v;
}

template <int D>
struct MmaCfg {
  static constexpr int HALF = D / 2;
  static constexpr int KS = D / 16;      // k-steps of the K-side product
  static constexpr int KW = D / 32;      // 32-bit words of K per thread per token (D/8 bytes)
  static constexpr int VB = D / 16;      // V bytes per thread per token
  static constexpr int VW = VB / 4;      // ... as full words
  static constexpr int VH = (VB % 4) / 2;  // ... plus half-words (D = 96)
  static constexpr int MB = VB;          // m-blocks of the V-side product
  static constexpr int DPT = D / 4;      // query dims held per thread
};

template <int D>
struct TileRegs {
  uint32_t k[2][MmaCfg<D>::KW];                       // tokens g, g+8
  uint32_t v[4][MmaCfg<D>::VW + MmaCfg<D>::VH];       // tokens 2c, 2c+1, 2c+8, 2c+9
  float kn[2], vn[2];                                 // norms of tokens g, g+8
  int pos0;                                           // absolute position of the tile's token 0
  uint32_t okmask;                                    // bit j: token j's page is valid
};

// byte offset (within a head's D/2 V bytes) of this thread's m-block i
template <int D>
__device__ __forceinline__ int v_byte_of_mblock(int g, int i) {
  using C = MmaCfg<D>;
  return i < 4 * C::VW ? g * 4 * C::VW + i : 32 * C::VW + 2 * g + (i - 4 * C::VW);
}

template <int D, int NB, bool ALIGNED, bool PAGE16, int WARPS>
__global__ void __launch_bounds__(WARPS * 32, 1) attention_mma_kernel(const AttnArgs a) {
  using C = MmaCfg<D>;
  const AttnShape& sh = a.sh;
  const AttnPlan& p = a.plan;
  extern __shared__ __align__(1024) unsigned char smem_raw[];
  const uint32_t base = smem_u32(smem_raw);
  const uint32_t tab = (base + (kTableBytes - 1)) & ~(kTableBytes - 1);
  if (tab + kTableBytes > base + kMmaSmemBytes) {  // cannot happen for a window base < 64 KB
    if (threadIdx.x == 0 && a.err_flag) atomicOr(a.err_flag, TQ4_DEV_TIMEOUT);
    return;
  }
  // ---- build the replicated byte -> half2 tables: slot l < 32 = K table of lane l, 32+l = V ----
  {
    uint32_t* t = reinterpret_cast<uint32_t*>(smem_raw + (tab - base));
    for (int i = threadIdx.x; i < 256 * 64; i += blockDim.x) {
      const int byte = i >> 6, slot = i & 63;
      const float* cent = slot < 32 ? a.k_centroids : a.v_centroids;
      const int nc = slot < 32 ? a.n_k_centroids : a.n_v_centroids;
      const float al = slot < 32 ? a.lut_scale_k : a.lut_scale_v;
      const int hi = byte >> 4, lo = byte & 15;
      t[i] = pack_h2(hi < nc ? __fmul_rn(al, cent[hi]) : 0.f, lo < nc ? __fmul_rn(al, cent[lo]) : 0.f);
    }
  }
  __syncthreads();

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, c = lane & 3;
  const uint32_t lb_k = tab + lane * 4, lb_v = tab + 128 + lane * 4;

  const int cta = blockIdx.x % sh.ctas, slice = blockIdx.x / sh.ctas;
  const int vh = slice * sh.HPC + warp % sh.HPC, ts = warp / sh.HPC;
  const int kvh = vh / sh.NCH, chunk = vh % sh.NCH;
  const int qh0 = kvh * sh.G + chunk * sh.GC;
  const int gcount = min(sh.GC, sh.G - chunk * sh.GC);
  const int total = p.scalars[0], tps = p.scalars[1];
  const int t_begin = cta * tps, t_end = min(total, t_begin + tps);
  if (t_begin >= t_end) return;
  const RowLayout lay = row_layout(sh.Hkv, D);
  const int k_off = lay.k_idx + kvh * C::HALF + c * (D / 8);
  const int kn_off = lay.k_norm + kvh * 4, vn_off = lay.v_norm + kvh * 4;
  const int v_off = lay.v_idx + kvh * C::HALF;

  int r;
  {
    int lo = 0, hi = sh.rows - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (p.tile_prefix[mid] <= t_begin) lo = mid; else hi = mid - 1;
    }
    r = lo;
    while (p.tile_prefix[r + 1] <= t_begin) ++r;
  }

  int t = t_begin;
  while (t < t_end) {
    const int row_t0 = p.tile_prefix[r], row_t1 = p.tile_prefix[r + 1];
    const int seg_end = min(row_t1, t_end);
    const int kv_start = p.kv_start[r], kv_end = p.kv_end[r];
    const int32_t* bt = a.block_table + (int64_t)p.row_seq[r] * a.bt_stride;
    const int tile0 = kv_start / kTileTokens;

    // ---- query fragments: column g of n-block nb = head nb*4 + g/2, term g%2 (hi / lo) ------
    uint32_t qf[NB][C::KS][2];
    float fscale[NB];  // qmax * sm_scale * log2(e) of head nb*4 + c
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
      // head nb*4 + c lives in column 2c: take its qmax from lane g' = 2c
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

    // ---- tile loader ---------------------------------------------------------------------
    auto row_offset = [&](int pos, bool& ok) -> int64_t {
      // byte offset of the token row at absolute position pos (clamped into the row's range)
      const int pc = min(max(pos, kv_start), kv_end - 1);
      const int blk = bt[pc / a.block_size];
      ok = blk >= 0 && blk < a.num_blocks;
      if (!ok && a.err_flag) atomicOr(a.err_flag, TQ4_DEV_BAD_BLOCK);
      return (int64_t)(ok ? blk : 0) * a.cache_block_stride +
             (int64_t)(pc % a.block_size) * a.cache_token_stride;
    };
    auto load_tile = [&](int tt, TileRegs<D>& R) {
      const int pos0 = (tile0 + (tt - row_t0)) * kTileTokens;
      R.pos0 = pos0;
      int64_t off_k0, off_k1, off_v[4];
      if (PAGE16) {
        bool ok;
        const int64_t b0 = row_offset(max(pos0, kv_start), ok) -
                           (int64_t)(max(pos0, kv_start) - pos0) * a.cache_token_stride;
        R.okmask = ok ? 0xFFFFu : 0u;
        off_k0 = b0 + (int64_t)g * a.cache_token_stride;
        off_k1 = off_k0 + 8 * a.cache_token_stride;
        off_v[0] = b0 + (int64_t)(2 * c) * a.cache_token_stride;
        off_v[1] = off_v[0] + a.cache_token_stride;
        off_v[2] = off_v[0] + 8 * a.cache_token_stride;
        off_v[3] = off_v[2] + a.cache_token_stride;
      } else {
        bool ok0, ok1, okv;
        off_k0 = row_offset(pos0 + g, ok0);
        off_k1 = row_offset(pos0 + g + 8, ok1);
        // every lane publishes the validity of tokens g and g+8; gather the 16-bit mask
        const uint32_t b0 = __ballot_sync(0xffffffffu, ok0), b1 = __ballot_sync(0xffffffffu, ok1);
        uint32_t mask = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) mask |= (((b0 >> (4 * j)) & 1u) << j) | (((b1 >> (4 * j)) & 1u) << (j + 8));
        R.okmask = mask;
        off_v[0] = row_offset(pos0 + 2 * c, okv);
        off_v[1] = row_offset(pos0 + 2 * c + 1, okv);
        off_v[2] = row_offset(pos0 + 2 * c + 8, okv);
        off_v[3] = row_offset(pos0 + 2 * c + 9, okv);
      }
      const uint8_t* k0 = a.cache + off_k0;
      const uint8_t* k1 = a.cache + off_k1;
      if (ALIGNED && C::KW % 4 == 0) {
#pragma unroll
        for (int w = 0; w < C::KW; w += 4) {
          ldg_stream_v4(k0 + k_off + 4 * w, R.k[0][w], R.k[0][w + 1], R.k[0][w + 2], R.k[0][w + 3]);
          ldg_stream_v4(k1 + k_off + 4 * w, R.k[1][w], R.k[1][w + 1], R.k[1][w + 2], R.k[1][w + 3]);
        }
      } else if (ALIGNED && C::KW % 2 == 0) {
#pragma unroll
        for (int w = 0; w < C::KW; w += 2) {
          ldg_stream_v2(k0 + k_off + 4 * w, R.k[0][w], R.k[0][w + 1]);
          ldg_stream_v2(k1 + k_off + 4 * w, R.k[1][w], R.k[1][w + 1]);
        }
      } else {
#pragma unroll
        for (int w = 0; w < C::KW; ++w) {
          R.k[0][w] = ldg_stream_b32(k0 + k_off + 4 * w);
          R.k[1][w] = ldg_stream_b32(k1 + k_off + 4 * w);
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint8_t* vp = a.cache + off_v[j] + v_off;
        if (ALIGNED && C::VW == 4) {
          ldg_stream_v4(vp + g * 16, R.v[j][0], R.v[j][1], R.v[j][2], R.v[j][3]);
        } else if (ALIGNED && C::VW == 2) {
          ldg_stream_v2(vp + g * 8, R.v[j][0], R.v[j][1]);
        } else {
#pragma unroll
          for (int w = 0; w < C::VW; ++w) R.v[j][w] = ldg_stream_b32(vp + g * 4 * C::VW + 4 * w);
        }
        if (C::VH) R.v[j][C::VW] = ldg_stream_b16(vp + 32 * C::VW + 2 * g);
      }
      R.kn[0] = ldg_f32(k0 + kn_off);
      R.kn[1] = ldg_f32(k1 + kn_off);
      R.vn[0] = ldg_f32(k0 + vn_off);
      R.vn[1] = ldg_f32(k1 + vn_off);
    };

    // ---- stream the segment's tiles ------------------------------------------------------------
    TileRegs<D> cur, nxt;
    int tt = t + ts;
    if (tt < seg_end) load_tile(tt, cur);
    for (; tt < seg_end; tt += sh.TPC) {
      const bool has_next = tt + sh.TPC < seg_end;
      if (has_next) load_tile(tt + sh.TPC, nxt);

      // K side: S^T = K * Qsplit^T
      float sacc[NB][4];
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.f;
#pragma unroll
      for (int w = 0; w < C::KW; ++w) {
        const uint32_t w0 = cur.k[0][w], w1 = cur.k[1][w];
        {
          const uint32_t a0 = lut<0>(w0, lb_k), a2 = lut<1>(w0, lb_k);
          const uint32_t a1 = lut<0>(w1, lb_k), a3 = lut<1>(w1, lb_k);
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) mma16816(sacc[nb], a0, a1, a2, a3, qf[nb][2 * w][0], qf[nb][2 * w][1]);
        }
        {
          const uint32_t a0 = lut<2>(w0, lb_k), a2 = lut<3>(w0, lb_k);
          const uint32_t a1 = lut<2>(w1, lb_k), a3 = lut<3>(w1, lb_k);
#pragma unroll
          for (int nb = 0; nb < NB; ++nb)
            mma16816(sacc[nb], a0, a1, a2, a3, qf[nb][2 * w + 1][0], qf[nb][2 * w + 1][1]);
        }
      }

      // softmax on (token g, head c) and (token g+8, head c)
      const int p0 = cur.pos0 + g, p1 = p0 + 8;
      const bool ok0 = p0 >= kv_start && p0 < kv_end && ((cur.okmask >> g) & 1u);
      const bool ok1 = p1 >= kv_start && p1 < kv_end && ((cur.okmask >> (g + 8)) & 1u);
      const float lg0 = ok0 ? fmaxf(log2f(cur.vn[0]), -30.f) : -CUDART_INF_F;
      const float lg1 = ok1 ? fmaxf(log2f(cur.vn[1]), -30.f) : -CUDART_INF_F;
      uint32_t pf[NB][2];
      float alpha[NB];
      bool rescale = false;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        const float s0 = ok0 ? (sacc[nb][0] + sacc[nb][1]) * (fscale[nb] * cur.kn[0]) : -CUDART_INF_F;
        const float s1 = ok1 ? (sacc[nb][2] + sacc[nb][3]) * (fscale[nb] * cur.kn[1]) : -CUDART_INF_F;
        float mt = fmaxf(s0 + lg0, s1 + lg1);
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 4));
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 8));
        mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 16));
        const float m_new = fmaxf(m[nb], mt);
        const float m_use = m_new == -CUDART_INF_F ? 0.f : m_new;
        alpha[nb] = exp2f(m[nb] - m_use);
        rescale |= (m_new != m[nb]);
        const float e0 = exp2f(s0 - m_use), e1 = exp2f(s1 - m_use);
        l[nb] = l[nb] * alpha[nb] + e0 + e1;
        m[nb] = m_new;
        const float w0 = ok0 ? e0 * cur.vn[0] : 0.f;
        const float w1 = ok1 ? e1 * cur.vn[1] : 0.f;
        pf[nb][0] = movmatrix_trans(split_h2(w0));
        pf[nb][1] = movmatrix_trans(split_h2(w1));
      }
      if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
          for (int i = 0; i < C::MB; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][nb][e] *= alpha[nb];
      }

      // V side: O^T += V^T * Psplit^T
#pragma unroll
      for (int w = 0; w < C::VW + C::VH; ++w) {
        const uint32_t x0 = cur.v[0][w], y0 = cur.v[1][w], x1 = cur.v[2][w], y1 = cur.v[3][w];
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
      if (has_next) cur = nxt;
    }

    // ---- write this warp's partial for the segment ---------------------------------------------
    const int slot = p.slot_base[r] + (cta - row_t0 / tps);
    const int64_t pidx = (int64_t)slot * sh.TPC + ts;
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
          p.part_m[hidx] = m[nb];
          p.part_l[hidx] = ls;
        }
        float* dst = p.part_o + hidx * D;
#pragma unroll
        for (int i = 0; i < C::MB; ++i) {
          const int vb = v_byte_of_mblock<D>(g, i);
          *reinterpret_cast<float2*>(dst + 2 * vb) =
              make_float2((acc[i][nb][0] + acc[i][nb][1]) * inv_av, (acc[i][nb][2] + acc[i][nb][3]) * inv_av);
        }
      }
    }
    t = seg_end;
    if (t < t_end) {
      ++r;
      while (p.tile_prefix[r + 1] <= t) ++r;
    }
  }
}

template <int D, int NB, bool ALIGNED, bool PAGE16>
int launch_mma_t(const AttnArgs& a, cudaStream_t st) {
  constexpr int WARPS = (D * NB <= 128) ? 16 : 8;
  auto kern = attention_mma_kernel<D, NB, ALIGNED, PAGE16, WARPS>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMmaSmemBytes) !=
        cudaSuccess)
      return TQ4_ERR_CUDA;
    attr_set = true;
  }
  const int warps = a.sh.HPC * a.sh.TPC;
  kern<<<a.sh.ctas * a.sh.n_slices, warps * 32, kMmaSmemBytes, st>>>(a);
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

template <int D, int NB>
int launch_mma_dn(const AttnArgs& a, cudaStream_t st) {
  const bool aligned = cache_aligned(a.sh, a.cache, a.cache_block_stride, a.cache_token_stride);
  const bool page16 = a.block_size % kTileTokens == 0;
  if (aligned && page16) return launch_mma_t<D, NB, true, true>(a, st);
  if (aligned) return launch_mma_t<D, NB, true, false>(a, st);
  if (page16) return launch_mma_t<D, NB, false, true>(a, st);
  return launch_mma_t<D, NB, false, false>(a, st);
}

template <int D>
int launch_mma_d(const AttnArgs& a, cudaStream_t st) {
  return a.sh.GC <= 4 ? launch_mma_dn<D, 1>(a, st) : launch_mma_dn<D, 2>(a, st);
}

}  // namespace

int mma_warps_per_cta(int D, int GC) { return (D * (GC <= 4 ? 1 : 2) <= 128) ? 16 : 8; }

bool attention_mma_supported(const AttnShape& sh, int block_size, const uint8_t* cache,
                             int64_t block_stride, int64_t token_stride) {
  (void)block_size; (void)cache; (void)block_stride;
  return supported_head_dim(sh.D) && sh.GC <= 8 && token_stride % 4 == 0;
}

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
