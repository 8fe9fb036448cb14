// Paged TQ4 attention: planning + query rotation, the fp32 CUDA-core streaming kernel,
// the split merge + un-rotation kernel, and the C entry points.
#include <math_constants.h>

#include <cstdlib>

#include "tq4_attention.cuh"

namespace tq4 {

// ======================================================================================
// 1. Prologue: q_rot = q * Pi^T for every (row, head), and (last block) the tile plan.
// ======================================================================================
// One block.  Phase 1 (inputs only, results in shared memory): per row the visible key range and
// its tile count, an exclusive scan of the tiles, the tiles per CTA, the partial slots per row and
// their scan.  Phase 2, after the preceding kernel has completed: the stores into the plan arrays.
// s_work: 2 * rows ints of dynamic shared memory.
__device__ void build_plan(const AttnArgs& a, int* s_work) {
  const AttnShape& sh = a.sh;
  const AttnPlan& p = a.plan;
  __shared__ int s_part[32];
  __shared__ int s_total;
  __shared__ int s_max_tiles;  // tiles of the longest row
  if (threadIdx.x == 0) s_max_tiles = 0;
  __syncthreads();
  const int rows = sh.rows;
  int* s_tiles = s_work;        // [rows] tile count, then exclusive prefix
  int* s_slots = s_work + rows; // [rows] slot count, then exclusive prefix
  const int per = (rows + blockDim.x - 1) / blockDim.x;
  const int r_lo = min(rows, (int)threadIdx.x * per), r_hi = min(rows, r_lo + per);

  auto row_range = [&](int r, int& seq, int& start, int& end) {
    const int gr = r + sh.row_offset;
    start = 0;
    end = 0;
    if (a.query_start_loc == nullptr) {
      seq = gr;
      if (seq < sh.num_seqs) {
        const int len = clamp_seq_len(a, max(0, a.seq_lens[seq]));
        end = len;
        start = a.sliding_window > 0 ? max(0, len - a.sliding_window) : 0;
      } else {
        seq = 0;
      }
    } else {
      // largest i with qsl[i] <= gr
      int lo = 0, hi = sh.num_seqs;  // qsl has num_seqs + 1 entries
      while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (a.query_start_loc[mid] <= gr) lo = mid; else hi = mid - 1;
      }
      seq = lo;
      if (seq < sh.num_seqs && gr < a.query_start_loc[sh.num_seqs]) {
        const int q0 = a.query_start_loc[seq], q1 = a.query_start_loc[seq + 1];
        const int len = clamp_seq_len(a, max(0, a.seq_lens[seq]));
        const int pos = len - (q1 - q0) + (gr - q0);
        end = a.causal ? pos + 1 : len;
        end = max(0, min(end, len));
        start = a.sliding_window > 0 ? max(0, pos + 1 - a.sliding_window) : 0;
        start = min(start, end);
      } else {
        seq = 0;
      }
    }
  };
  // exclusive scan over the block's threads (shuffle scan per warp + scan of the warp totals);
  // s_total receives the sum
  auto block_exclusive_scan = [&](int mine) -> int {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    int incl = mine;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    if (lane == 31) s_part[wid] = incl;
    __syncthreads();
    if (wid == 0) {
      const int tot = lane < nw ? s_part[lane] : 0;
      int winc = tot;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int up = __shfl_up_sync(0xffffffffu, winc, o);
        if (lane >= o) winc += up;
      }
      if (lane < nw) s_part[lane] = winc - tot;  // exclusive warp offsets
      if (lane == 31) s_total = winc;
    }
    __syncthreads();
    const int base = s_part[wid] + incl - mine;
    __syncthreads();
    return base;
  };

  int local = 0, row_max = 0;
  for (int r = r_lo; r < r_hi; ++r) {
    int seq, start, end;
    row_range(r, seq, start, end);
    const int nt = end > start ? (end + kTileTokens - 1) / kTileTokens - start / kTileTokens : 0;
    s_tiles[r] = nt;
    local += nt;
    row_max = max(row_max, nt);
  }
  if (row_max > 0) atomicMax(&s_max_tiles, row_max);
  int run = block_exclusive_scan(local);
  for (int r = r_lo; r < r_hi; ++r) {
    const int nt = s_tiles[r];
    s_tiles[r] = run;
    run += nt;
  }
  const int total = s_total;
  const int tps = tiles_per_span(total, sh.span_ctas, s_max_tiles);
  __syncthreads();
  local = 0;
  for (int r = r_lo; r < r_hi; ++r) {
    const int b = s_tiles[r];
    const int e = r + 1 < rows ? s_tiles[r + 1] : total;
    const int n = e > b ? (e - 1) / tps - b / tps + 1 : 0;
    s_slots[r] = n;
    local += n;
  }
  __syncthreads();
  run = block_exclusive_scan(local);
  const int total_slots = s_total;

  pdl_wait();
  for (int r = r_lo; r < r_hi; ++r) {
    int seq, start, end;
    row_range(r, seq, start, end);
    p.kv_start[r] = start;
    p.kv_end[r] = end;
    p.row_seq[r] = seq;
    p.tile_prefix[r] = s_tiles[r];
    p.slot_base[r] = run;
    run += s_slots[r];
  }
  if (threadIdx.x == 0) {
    p.tile_prefix[rows] = total;
    p.scalars[0] = total;
    p.scalars[1] = tps;
    p.slot_base[rows] = total_slots;
  }
}

template <int D>
struct QrotCfg {
  static constexpr int DC = D < 128 ? D : 128;          // columns of Pi staged per pass
  static constexpr int G = 256 / D >= 1 ? 256 / D : 1;  // thread groups (one output column each)
  static constexpr int VPG = 4;                         // vectors per group (small: many blocks)
  static constexpr int VB = G * VPG;                    // (row, head) vectors per block
  static constexpr int THREADS = G * D;
  static constexpr size_t rot_bytes = ((size_t)D * (DC + 1) + (size_t)D * VB) * sizeof(float);
  static constexpr size_t plan_bytes = 2 * (size_t)kMaxRowsPerLaunch * sizeof(int);  // planning block
  static constexpr size_t smem_bytes = rot_bytes > plan_bytes ? rot_bytes : plan_bytes;
};

// q_rot[v][j] = sum_d q[v][d] * Pi[j][d].  Pi is staged once per block, transposed into a padded
// shared array so that thread j walks its own row without bank conflicts; the block's vectors sit
// in shared memory as [d][v] (swizzled) so that one 16-byte broadcast load feeds four FMAs.
template <int D>
__global__ void __launch_bounds__(QrotCfg<D>::THREADS) qrot_plan_kernel(const AttnArgs a) {
  using Q = QrotCfg<D>;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_trigger();
  if (blockIdx.x == gridDim.x - 1) {  // the planning block
    build_plan(a, reinterpret_cast<int*>(smem_raw));
    return;
  }
  constexpr int DC = Q::DC, VB = Q::VB, VPG = Q::VPG, PITCH = DC + 1;
  float* s_pi = reinterpret_cast<float*>(smem_raw);  // [D][DC + 1]
  float* s_q = s_pi + D * PITCH;                     // [D][VB], v swizzled by d
  const AttnShape& sh = a.sh;
  const int64_t n_vec = (int64_t)sh.rows * sh.Hq;
  const int64_t v0 = (int64_t)blockIdx.x * VB;
  const int tid = threadIdx.x, grp = tid / D, j = tid - grp * D;
  auto swz = [](int d) { return ((d & 7) << 2) & (VB - 1); };

  // the block's vectors (coalesced over d), converted to fp32
  for (int i0 = 0; i0 < VB * D; i0 += Q::THREADS * 8) {
    float x[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * Q::THREADS + tid;
      const int v = i / D, d = i - v * D;
      const int64_t vec = v0 + v;
      x[u] = 0.f;
      if (i < VB * D && vec < n_vec) {
        const int64_t row = vec / sh.Hq + sh.row_offset;
        const int h = (int)(vec % sh.Hq);
        x[u] = load_as_float(a.q, a.q_dtype, row * a.q_token_stride + h * a.q_head_stride + d);
      }
    }
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int i = i0 + u * Q::THREADS + tid;
      const int v = i / D, d = i - v * D;
      if (i < VB * D) s_q[d * VB + (v ^ swz(d))] = x[u];
    }
  }

  float acc[VPG];
#pragma unroll
  for (int v = 0; v < VPG; ++v) acc[v] = 0.f;
  for (int d0 = 0; d0 < D; d0 += DC) {
    __syncthreads();
    // stage Pi[:, d0 : d0 + DC] with 16-byte loads, eight in flight per thread
    constexpr int N4 = D * DC / 4;
    for (int i0 = 0; i0 < N4; i0 += Q::THREADS * 8) {
      float4 x[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * Q::THREADS + tid;
        if (i < N4) {
          const int jj = i / (DC / 4), c4 = i - jj * (DC / 4);
          x[u] = __ldg(reinterpret_cast<const float4*>(a.rotation + (size_t)jj * D + d0) + c4);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * Q::THREADS + tid;
        if (i < N4) {
          const int jj = i / (DC / 4), c4 = i - jj * (DC / 4);
          float* dst = s_pi + jj * PITCH + 4 * c4;
          dst[0] = x[u].x; dst[1] = x[u].y; dst[2] = x[u].z; dst[3] = x[u].w;
        }
      }
    }
    __syncthreads();
#pragma unroll 4
    for (int dd = 0; dd < DC; ++dd) {
      const float pv = s_pi[j * PITCH + dd];
      const int d = d0 + dd;
      const float* qrow = s_q + d * VB;
#pragma unroll
      for (int v4 = 0; v4 < VPG / 4; ++v4) {
        const float4 qv = *reinterpret_cast<const float4*>(qrow + ((grp * VPG + 4 * v4) ^ swz(d)));
        acc[4 * v4] = fmaf(qv.x, pv, acc[4 * v4]);
        acc[4 * v4 + 1] = fmaf(qv.y, pv, acc[4 * v4 + 1]);
        acc[4 * v4 + 2] = fmaf(qv.z, pv, acc[4 * v4 + 2]);
        acc[4 * v4 + 3] = fmaf(qv.w, pv, acc[4 * v4 + 3]);
      }
    }
  }
  pdl_wait();  // the scratch may still be read by the attention kernel of the previous call
#pragma unroll
  for (int v = 0; v < VPG; ++v) {
    const int64_t vec = v0 + grp * VPG + v;
    if (vec < n_vec) a.plan.q_rot[vec * D + j] = acc[v];
  }
}

// --------------------------------------------------------------------------------------
// Fused prologue (head_dim <= 128): ONE launch rotates every query vector of the call and, when
// the call carries new tokens, compresses their K and V vectors into the paged cache; an extra
// block builds the tile plan.  Pi^T is staged once per block into shared memory ([d][j]); one WARP
// handles four vectors at a time as a 4 x D strip of the product X * Pi^T, each lane a 4 x 4
// register tile (four vectors x four consecutive output coordinates), so a step of the reduction
// is two 16-byte shared loads and 16 FMAs, and nothing but warp-level synchronisation is needed.
//
// The write part keeps the arithmetic contract of the compress kernels bit for bit
// (tq4_compress.cu): squared norm by lane-strided FMAs + butterfly reduction, IEEE division by
// (norm + 1e-10), four quarter-length FMA chains in ascending k combined as (s0 + s1) + (s2 + s3).
// --------------------------------------------------------------------------------------
template <int D>
struct PrologueCfg {
  static constexpr int WARPS = 8;
  static constexpr int THREADS = WARPS * 32;
  static constexpr int VC = 4;            // vectors per warp per pass
  static constexpr size_t rot_bytes = ((size_t)D * D + (size_t)WARPS * D * VC) * sizeof(float);
  static constexpr size_t plan_bytes = 2 * (size_t)kMaxRowsPerLaunch * sizeof(int);
  static constexpr size_t smem_bytes = rot_bytes > plan_bytes ? rot_bytes : plan_bytes;
};

template <int D>
__global__ void __launch_bounds__(PrologueCfg<D>::THREADS)
prologue_kernel(const AttnArgs a, const CompressArgs w, const int has_attn, const int has_write) {
  using P = PrologueCfg<D>;
  constexpr int VC = P::VC, HALF = D / 2, KQ = D / 4, XPL = D / 32;
  static_assert(D % 32 == 0 && D <= 128 && KQ % 8 == 0, "head_dim must be a multiple of 32, at most 128");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_trigger();
  if (has_attn && blockIdx.x == gridDim.x - 1) {  // the planning block
    build_plan(a, reinterpret_cast<int*>(smem_raw));
    return;
  }
  const int n_rot_blocks = (int)gridDim.x - (has_attn ? 1 : 0);
  float* s_pit = reinterpret_cast<float*>(smem_raw);                    // [D][D]: s_pit[d][j] = Pi[j][d]
  float4* s_x = reinterpret_cast<float4*>(s_pit + D * D);               // [WARPS][D] four vectors per entry
  __shared__ float s_bounds[2][16];  // sorted boundaries of K and V, padded with +inf
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (has_write && tid < 32) {
    const int src = tid >> 4, i = tid & 15;
    s_bounds[src][i] = (src < w.n_sources && i < w.n_bounds[src]) ? w.bounds[src][i] : CUDART_INF_F;
  }

  // ---- stage Pi^T ------------------------------------------------------------------------------
  if (has_attn) {
    // thread -> (4 consecutive d of row j), consecutive threads = consecutive j: conflict-free stores
    constexpr int N4 = D * D / 4;
    for (int i0 = 0; i0 < N4; i0 += P::THREADS * 8) {
      float4 x[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * P::THREADS + tid;
        const int c4 = i / D, jj = i - c4 * D;
        if (i < N4) x[u] = __ldg(reinterpret_cast<const float4*>(a.rotation + (size_t)jj * D) + c4);
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * P::THREADS + tid;
        const int c4 = i / D, jj = i - c4 * D;
        if (i < N4) {
          float* dst = s_pit + (4 * c4) * D + jj;
          dst[0] = x[u].x; dst[D] = x[u].y; dst[2 * D] = x[u].z; dst[3 * D] = x[u].w;
        }
      }
    }
  } else {  // write only: the caller gave Pi^T split into even / odd output columns
    for (int i = tid; i < D * HALF; i += P::THREADS) {
      const int k = i / HALF, pp = i - k * HALF;
      s_pit[k * D + 2 * pp] = __ldg(w.rot_even + i);
      s_pit[k * D + 2 * pp + 1] = __ldg(w.rot_odd + i);
    }
  }
  __syncthreads();

  // vector counts fit 32 bits (rows <= kMaxRowsPerLaunch, writes <= kSmallRows): no 64-bit divisions
  const int n_q = has_attn ? a.sh.rows * a.sh.Hq : 0;
  const int rows_per_src = has_write ? (int)w.n_tokens * w.num_heads : 0;
  const int n_w = rows_per_src * (has_write ? w.n_sources : 0);
  const int cq = (n_q + VC - 1) / VC, cw = (n_w + VC - 1) / VC;
  float4* gx = s_x + warp * D;
  const bool jact = 4 * lane < D;                       // this lane owns outputs 4*lane .. 4*lane+3
  const float4* pcol = reinterpret_cast<const float4*>(s_pit) + (jact ? lane : 0);  // + d * (D/4)
  // (source, token, head) of write vector `vec`
  auto w_coords = [&](int vec, int& src, int& tok, int& h) {
    src = vec >= rows_per_src ? 1 : 0;
    const unsigned rem = (unsigned)(vec - src * rows_per_src);
    tok = (int)(rem / (unsigned)w.num_heads);
    h = (int)(rem - (unsigned)tok * (unsigned)w.num_heads);
  };

  for (int c = (int)blockIdx.x * P::WARPS + warp; c < cq + cw; c += n_rot_blocks * P::WARPS) {
    const bool is_w = c >= cq;
    const int v0 = (is_w ? c - cq : c) * VC;
    const int nv = is_w ? n_w : n_q;
    // ---- load: lane l holds elements l, l+32, ... of each of the four vectors -------------------
    float xr[XPL][VC];
    const int dt = is_w ? w.x_dtype : a.q_dtype;
    const void* base[VC];
#pragma unroll
    for (int v = 0; v < VC; ++v) {
      const int vec = v0 + v;
      base[v] = nullptr;
      if (vec < nv) {
        if (!is_w) {
          const unsigned rr = (unsigned)vec / (unsigned)a.sh.Hq;
          const int h = (int)((unsigned)vec - rr * (unsigned)a.sh.Hq);
          base[v] = byte_offset(a.q, dt, ((int64_t)rr + a.sh.row_offset) * a.q_token_stride +
                                             h * a.q_head_stride + lane);
        } else {
          int src, tok, h;
          w_coords(vec, src, tok, h);
          base[v] = byte_offset(w.x[src], dt, (int64_t)tok * w.token_stride[src] +
                                                  (int64_t)h * w.head_stride[src] + lane);
        }
      }
    }
    if (dt == TQ4_F32) load_strip<float, XPL, VC>(base, xr);
    else if (dt == TQ4_F16) load_strip<__half, XPL, VC>(base, xr);
    else load_strip<__nv_bfloat16, XPL, VC>(base, xr);
    float nrm[VC];
    if (is_w) {
#pragma unroll
      for (int v = 0; v < VC; ++v) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < XPL; ++i) ss = fmaf(xr[i][v], xr[i][v], ss);
        nrm[v] = sqrtf(warp_sum(ss));
        const float den = nrm[v] + 1e-10f;
#pragma unroll
        for (int i = 0; i < XPL; ++i) xr[i][v] = xr[i][v] / den;
      }
    }
    __syncwarp();  // the previous pass has finished reading the staging strip
#pragma unroll
    for (int i = 0; i < XPL; ++i) gx[lane + 32 * i] = make_float4(xr[i][0], xr[i][1], xr[i][2], xr[i][3]);
    __syncwarp();

    // ---- y[v][4*lane + jj] = sum_d x[v][d] * Pi[4*lane + jj][d] as (s0 + s1) + (s2 + s3): the two
    // quarter chains of a half advance together (32 independent accumulators); loops stay rolled,
    // a launch of a few thousand vectors runs this code once per warp and pays for its size
    float y[VC][4];
#pragma unroll 1
    for (int hf = 0; hf < 2; ++hf) {
      float sa[VC][4], sb[VC][4];
#pragma unroll
      for (int v = 0; v < VC; ++v)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) sa[v][jj] = sb[v][jj] = 0.f;
      const float4* pa = pcol + (2 * hf) * KQ * (D / 4);
      const float4* xa = gx + (2 * hf) * KQ;
#pragma unroll 4
      for (int dd = 0; dd < KQ; ++dd) {
        const float4 p0 = pa[dd * (D / 4)], x0 = xa[dd];
        const float4 p1 = pa[(KQ + dd) * (D / 4)], x1 = xa[KQ + dd];
        const float xs0[VC] = {x0.x, x0.y, x0.z, x0.w}, ps0[4] = {p0.x, p0.y, p0.z, p0.w};
        const float xs1[VC] = {x1.x, x1.y, x1.z, x1.w}, ps1[4] = {p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int v = 0; v < VC; ++v)
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            sa[v][jj] = fmaf(xs0[v], ps0[jj], sa[v][jj]);
            sb[v][jj] = fmaf(xs1[v], ps1[jj], sb[v][jj]);
          }
      }
#pragma unroll
      for (int v = 0; v < VC; ++v)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj)
          y[v][jj] = hf == 0 ? sa[v][jj] + sb[v][jj] : y[v][jj] + (sa[v][jj] + sb[v][jj]);
    }

    pdl_wait();  // nothing before this point wrote global memory
    if (!is_w) {
#pragma unroll
      for (int v = 0; v < VC; ++v)
        if (v0 + v < nv && jact)
          *reinterpret_cast<float4*>(a.plan.q_rot + (int64_t)(v0 + v) * D + 4 * lane) =
              make_float4(y[v][0], y[v][1], y[v][2], y[v][3]);
    } else {
      const RowLayout lay = row_layout(w.num_heads, D);
#pragma unroll
      for (int v = 0; v < VC; ++v) {
        const int vec = v0 + v;
        if (vec >= nv) continue;
        int src, tok, h;
        w_coords(vec, src, tok, h);
        const float* bd = s_bounds[src];
        const unsigned b0 = (unsigned)((bucketize_sorted16(y[v][0], bd) << 4) | bucketize_sorted16(y[v][1], bd));
        const unsigned b1 = (unsigned)((bucketize_sorted16(y[v][2], bd) << 4) | bucketize_sorted16(y[v][3], bd));
        uint8_t* dst_idx;
        float* dst_norm;
        if (w.cache != nullptr) {
          if (tok >= w.n_slots) continue;
          const int64_t slot = w.slot_mapping[tok];
          if (slot < 0) continue;
          if (slot >= w.num_cache_slots) {
            if (lane == 0 && w.err_flag) atomicOr(w.err_flag, TQ4_DEV_BAD_SLOT);
            continue;
          }
          uint8_t* rowp = w.cache + slot * w.cache_token_stride;
          dst_idx = rowp + (src == 0 ? lay.k_idx : lay.v_idx) + h * HALF;
          dst_norm = reinterpret_cast<float*>(rowp + (src == 0 ? lay.k_norm : lay.v_norm) + h * 4);
        } else {
          dst_idx = w.packed_out + (int64_t)vec * HALF;
          dst_norm = w.norms_out + vec;
        }
        // bytes 2*lane, 2*lane+1 of the head's packed row (2-byte aligned: rows start on 4 bytes)
        if (jact) *reinterpret_cast<uint16_t*>(dst_idx + 2 * lane) = (uint16_t)(b0 | (b1 << 8));
        if (lane == 0) *dst_norm = nrm[v];
      }
    }
  }
  pdl_wait();
}

template <int D>
int launch_prologue_t(const AttnArgs* a, const CompressArgs* w, cudaStream_t st) {
  using P = PrologueCfg<D>;
  if (!ensure_dynamic_smem<prologue_kernel<D>>((int)P::smem_bytes, true)) return TQ4_ERR_CUDA;
  const int64_t n_q = a ? (int64_t)a->sh.rows * a->sh.Hq : 0;
  const int64_t n_w = w ? w->n_tokens * w->num_heads * w->n_sources : 0;
  const int64_t chunks = (n_q + P::VC - 1) / P::VC + (n_w + P::VC - 1) / P::VC;
  int64_t blocks = (chunks + P::WARPS - 1) / P::WARPS;
  if (blocks > 2 * (int64_t)sm_count()) blocks = 2 * (int64_t)sm_count();
  if (blocks < 1) blocks = 1;
  static const AttnArgs no_attn{};
  static const CompressArgs no_write{};
  // First kernel of an entry point: a plain stream-ordered launch.  It reads tensors the caller's
  // preceding kernel may have produced (q, key, value, seq_lens), so it must not start before that
  // kernel has completed, whatever launch style the caller's kernels use.
  if (launch_kernel(prologue_kernel<D>, dim3((unsigned)blocks + (a ? 1 : 0)), dim3(P::THREADS), P::smem_bytes,
                    st, false, a ? *a : no_attn, w ? *w : no_write, a ? 1 : 0, w ? 1 : 0) != cudaSuccess)
    return TQ4_ERR_CUDA;
  TQ4_CHECK_LAUNCH();
  return TQ4_OK;
}

// ======================================================================================
// 2. fp32 CUDA-core streaming kernel (any supported head_dim, any group size).
// ======================================================================================
template <int D, int GC>
struct Fp32Cfg {
  static constexpr int REPS = (D + 127) / 128;  // 4-dim groups per lane in the V phase
  static constexpr int KW = D / 16;             // 32-bit words of K per lane (half a row)
  static constexpr size_t smem_per_warp =
      (size_t)GC * D * 4 + kTileTokens * GC * 4 + kTileTokens * 8;
};

template <int D, int GC>
__global__ void __launch_bounds__(kMaxWarpsPerCta * 32)
attention_fp32_kernel(const AttnArgs a) {
  using Cfg = Fp32Cfg<D, GC>;
  constexpr int REPS = Cfg::REPS, KW = Cfg::KW, HALF = D / 2;
  const AttnShape& sh = a.sh;
  const AttnPlan& p = a.plan;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __shared__ float lut_k[TQ4_MAX_CENTROIDS], lut_v[TQ4_MAX_CENTROIDS];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  unsigned char* wbase = smem_raw + warp * Cfg::smem_per_warp;
  float* s_q = reinterpret_cast<float*>(wbase);                       // [GC][D]
  float* s_p = s_q + GC * D;                                          // [16][GC]  p * vnorm
  int64_t* s_row = reinterpret_cast<int64_t*>(s_p + kTileTokens * GC);  // [16] row byte offset, -1 = masked

  if (threadIdx.x < TQ4_MAX_CENTROIDS) {
    lut_k[threadIdx.x] = threadIdx.x < a.n_k_centroids ? a.k_centroids[threadIdx.x] : 0.f;
    lut_v[threadIdx.x] = threadIdx.x < a.n_v_centroids ? a.v_centroids[threadIdx.x] : 0.f;
  }
  __syncthreads();
  pdl_trigger();
  pdl_wait();  // plan, rotated queries and cache come from the preceding kernels

  const int c = blockIdx.x % sh.ctas, slice = blockIdx.x / sh.ctas;
  const int vh = slice * sh.HPC + warp % sh.HPC, ts = warp / sh.HPC;
  const int kvh = vh / sh.NCH, chunk = vh % sh.NCH;
  const int qh0 = kvh * sh.G + chunk * sh.GC;
  const int gcount = min(sh.GC, sh.G - chunk * sh.GC);
  const int total = p.scalars[0], tps = p.scalars[1];
  const int t_begin = c * tps, t_end = min(total, t_begin + tps);
  if (t_begin >= t_end) return;
  const RowLayout lay = row_layout(sh.Hkv, D);

  // first row r with tile_prefix[r] <= t_begin < tile_prefix[r+1]
  int r;
  {
    int lo = 0, hi = sh.rows - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (p.tile_prefix[mid] <= t_begin) lo = mid; else hi = mid - 1;
    }
    r = lo;
    while (p.tile_prefix[r + 1] <= t_begin) ++r;  // skip rows without tiles
  }
  const int tok = lane & 15, half = lane >> 4;

  int t = t_begin;
  while (t < t_end) {
    const int row_t0 = p.tile_prefix[r], row_t1 = p.tile_prefix[r + 1];
    const int seg_end = min(row_t1, t_end);
    const int kv_start = p.kv_start[r], kv_end = p.kv_end[r];
    const int32_t* bt = a.block_table + (int64_t)p.row_seq[r] * a.bt_stride;
    const int tile0 = kv_start / kTileTokens;  // absolute tile index of the row's first tile

    // q of this row's heads -> smem
    __syncwarp();
    for (int i = lane; i < GC * D; i += 32) {
      const int g = i / D, d = i - g * D;
      s_q[i] = g < gcount ? p.q_rot[((int64_t)r * sh.Hq + qh0 + g) * D + d] : 0.f;
    }
    __syncwarp();

    float m[GC], l[GC], acc[GC][REPS][4];
#pragma unroll
    for (int g = 0; g < GC; ++g) {
      m[g] = -CUDART_INF_F;
      l[g] = 0.f;
#pragma unroll
      for (int rep = 0; rep < REPS; ++rep)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[g][rep][e] = 0.f;
    }

    for (int tt = t + ts; tt < seg_end; tt += sh.TPC) {
      const int pos = (tile0 + (tt - row_t0)) * kTileTokens + tok;
      // ---- K phase: lane = (half, token) -------------------------------------------------
      int64_t row_off = -1;
      if (pos >= kv_start && pos < kv_end) {
        const int blk = bt[pos / a.block_size];
        if (blk < 0 || blk >= a.num_blocks) {
          if (a.err_flag) atomicOr(a.err_flag, TQ4_DEV_BAD_BLOCK);
        } else {
          row_off = (int64_t)blk * a.cache_block_stride +
                    (int64_t)(pos % a.block_size) * a.cache_token_stride;
        }
      }
      float dot[GC];
#pragma unroll
      for (int g = 0; g < GC; ++g) dot[g] = 0.f;
      float knorm = 0.f, vnorm = 0.f;
      if (row_off >= 0) {
        const uint8_t* rowp = a.cache + row_off;
        const uint32_t* kw = reinterpret_cast<const uint32_t*>(rowp + lay.k_idx + kvh * HALF + half * (HALF / 2));
        knorm = *reinterpret_cast<const float*>(rowp + lay.k_norm + kvh * 4);
        vnorm = *reinterpret_cast<const float*>(rowp + lay.v_norm + kvh * 4);
        const int dbase = half * HALF;
#pragma unroll
        for (int w = 0; w < KW; ++w) {
          const uint32_t word = kw[w];
#pragma unroll
          for (int b = 0; b < 4; ++b) {
            const uint32_t byte = (word >> (8 * b)) & 0xFFu;
            const float ce = lut_k[byte >> 4], co = lut_k[byte & 0xFu];
            const int d = dbase + w * 8 + b * 2;
#pragma unroll
            for (int g = 0; g < GC; ++g) {
              dot[g] = fmaf(s_q[g * D + d], ce, dot[g]);
              dot[g] = fmaf(s_q[g * D + d + 1], co, dot[g]);
            }
          }
        }
      }
      if (half == 0) s_row[tok] = row_off;
      float pw[GC];
#pragma unroll
      for (int g = 0; g < GC; ++g) {
        float s = dot[g] + __shfl_xor_sync(0xffffffffu, dot[g], 16);
        s = row_off >= 0 ? s * knorm * a.scale_log2e : -CUDART_INF_F;
        float mt = s;
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, o));
        const float m_new = fmaxf(m[g], mt);
        const float m_use = m_new == -CUDART_INF_F ? 0.f : m_new;
        const float alpha = exp2f(m[g] - m_use);
        const float pr = exp2f(s - m_use);
        m[g] = m_new;
        l[g] = l[g] * alpha + (half == 0 ? pr : 0.f);
        pw[g] = pr * vnorm;
#pragma unroll
        for (int rep = 0; rep < REPS; ++rep)
#pragma unroll
          for (int e = 0; e < 4; ++e) acc[g][rep][e] *= alpha;
      }
      if (half == 0) {
#pragma unroll
        for (int g = 0; g < GC; ++g) s_p[tok * GC + g] = pw[g];
      }
      __syncwarp();
      // ---- V phase: lane = 4 consecutive dims per rep -----------------------------------
#pragma unroll 4
      for (int tk = 0; tk < kTileTokens; ++tk) {
        const int64_t ro = s_row[tk];
        if (ro < 0) continue;
        const uint8_t* vrow = a.cache + ro + lay.v_idx + kvh * HALF;
#pragma unroll
        for (int rep = 0; rep < REPS; ++rep) {
          const int byte0 = 2 * (lane + 32 * rep);
          if (byte0 < HALF) {
            const uint32_t hv = *reinterpret_cast<const uint16_t*>(vrow + byte0);
            const float c0 = lut_v[(hv >> 4) & 0xFu], c1 = lut_v[hv & 0xFu];
            const float c2 = lut_v[(hv >> 12) & 0xFu], c3 = lut_v[(hv >> 8) & 0xFu];
#pragma unroll
            for (int g = 0; g < GC; ++g) {
              const float w = s_p[tk * GC + g];
              acc[g][rep][0] = fmaf(w, c0, acc[g][rep][0]);
              acc[g][rep][1] = fmaf(w, c1, acc[g][rep][1]);
              acc[g][rep][2] = fmaf(w, c2, acc[g][rep][2]);
              acc[g][rep][3] = fmaf(w, c3, acc[g][rep][3]);
            }
          }
        }
      }
      __syncwarp();
    }

    // ---- write this warp's partial for the segment ---------------------------------------
    const int slot = p.slot_base[r] + (c - row_t0 / tps);
    const int64_t pidx = (int64_t)slot * sh.TPC + ts;
#pragma unroll
    for (int g = 0; g < GC; ++g) {
      if (g < gcount) {
        const float lsum = warp_sum(l[g]);
        const int64_t hidx = pidx * sh.Hq + qh0 + g;
        if (lane == 0) {
          p.part_m[hidx] = m[g];
          p.part_l[hidx] = lsum;
        }
#pragma unroll
        for (int rep = 0; rep < REPS; ++rep) {
          const int d = 4 * (lane + 32 * rep);
          if (d < D)
            *reinterpret_cast<float4*>(p.part_o + hidx * D + d) =
                make_float4(acc[g][rep][0], acc[g][rep][1], acc[g][rep][2], acc[g][rep][3]);
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

template <int D, int GC>
int launch_fp32_t(const AttnArgs& a, cudaStream_t st) {
  using Cfg = Fp32Cfg<D, GC>;
  const size_t smem = Cfg::smem_per_warp * kMaxWarpsPerCta;
  if (!ensure_dynamic_smem<attention_fp32_kernel<D, GC>>((int)smem)) return TQ4_ERR_CUDA;
  const int warps = a.sh.HPC * a.sh.TPC;
  if (launch_kernel(attention_fp32_kernel<D, GC>, dim3(a.sh.ctas * a.sh.n_slices), dim3(warps * 32), smem, st,
                    true, a) != cudaSuccess)
    return TQ4_ERR_CUDA;
  TQ4_CHECK_LAUNCH();
  return TQ4_OK;
}

template <int D>
int launch_fp32_d(const AttnArgs& a, cudaStream_t st) {
  const int gc = a.sh.GC;
  if (gc <= 1) return launch_fp32_t<D, 1>(a, st);
  if (gc <= 2) return launch_fp32_t<D, 2>(a, st);
  if (gc <= 4) return launch_fp32_t<D, 4>(a, st);
  return launch_fp32_t<D, 8>(a, st);
}

int launch_attention_fp32(const AttnArgs& a, cudaStream_t st) {
  switch (a.sh.D) {
    case 64: return launch_fp32_d<64>(a, st);
    case 96: return launch_fp32_d<96>(a, st);
    case 128: return launch_fp32_d<128>(a, st);
    case 256: return launch_fp32_d<256>(a, st);
  }
  return TQ4_ERR_UNSUPPORTED;
}

// ======================================================================================
// 3. Merge the partials of a row, normalise, un-rotate, store.
//    Also serves tq4_combine_partials (cross-GPU shards) through the "dense" mode.
// ======================================================================================
constexpr int kCombHeads = 8;

struct CombineArgs {
  // sparse mode (plan != null): slots of row r are slot_base[r]..slot_base[r+1], x TPC
  const int* slot_base;
  int TPC;
  const float* part_o;
  const float* part_m;
  const float* part_l;
  // dense mode (slot_base == null): `world` parts, part index w*rows + r; part_m holds natural-log
  // LSE and part_o is already normalised
  int world;
  int rows, row_offset, Hq;
  const float* rotation;
  void* out;
  int out_dtype;
  int64_t out_token_stride, out_head_stride;
  float* lse_out;
  int out_rotated;
};

constexpr int kCombMaxParts = 64;  // partials of one row merged per pass

constexpr int kCombFastParts = 8;   // up to this many partials per vector take the one-round-trip path

// Batches of 8 consecutive (row, head) vectors, D threads, a block walks batches grid-stride.
// Pi is copied to shared memory asynchronously at kernel entry (once per block) and overlaps the
// merge of the partials.  Typical decode rows have at most 8 partials: then every load of a batch
// (8 x 8 accumulator elements per thread, the 64 maxima and sums by the first 64 threads) is issued
// before anything is consumed, so a batch costs two dependent memory round trips.  Rows with more
// partials go through passes of 64 partials with the merge weights staged in shared memory.
template <int D>
__global__ void __launch_bounds__(D) combine_kernel(const CombineArgs a) {
  static_assert(D >= kCombHeads * kCombFastParts, "the fast path loads one (vector, partial) pair per thread");
  extern __shared__ __align__(16) unsigned char smem_raw[];
  float* s_pi = reinterpret_cast<float*>(smem_raw);            // [D][D] (D <= 128 only)
  float* s_o = s_pi + (D <= 128 ? D * D : 0);                   // [D][kCombHeads]
  float* s_w = s_o + kCombHeads * D;                            // [kCombMaxParts][kCombHeads]
  float* s_m = s_w + kCombMaxParts * kCombHeads;                // [kCombHeads] running max
  float* s_l = s_m + kCombHeads;                                // [kCombHeads] running sum
  __shared__ long long s_p0[kCombHeads];                        // first partial of the vector's row
  __shared__ int s_np[kCombHeads], s_row[kCombHeads], s_head[kCombHeads];
  const int d = threadIdx.x;
  const int64_t n_vec = (int64_t)a.rows * a.Hq;
  const int64_t n_batches = (n_vec + kCombHeads - 1) / kCombHeads;
  constexpr float kLn2 = 0.6931471805599453f, kLog2e = 1.4426950408889634f;
  constexpr bool kStagePi = D <= 128;  // a 256 x 256 fp32 Pi does not fit in shared memory
  if (kStagePi && !a.out_rotated) {
    const uint32_t dst = (uint32_t)__cvta_generic_to_shared(s_pi);
    for (int i = d; i < D * D / 4; i += D)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + i * 16),
                   "l"(a.rotation + (size_t)i * 4) : "memory");
    asm volatile("cp.async.commit_group;" ::: "memory");
  }
  pdl_wait();  // the partials and the plan come from the kernels before this one
  const bool sparse = a.slot_base != nullptr;
  const float mscale = sparse ? 1.f : kLog2e;  // dense partials carry a natural-log LSE
  const int64_t pstride = (sparse ? (int64_t)1 : (int64_t)a.rows) * a.Hq * D;

  for (int64_t batch = blockIdx.x; batch < n_batches; batch += gridDim.x) {
    const int64_t v0 = batch * kCombHeads;
    const int nh = (int)min((int64_t)kCombHeads, n_vec - v0);
    if (d < kCombHeads) {
      const int64_t v = v0 + d;
      const int r = d < nh ? (int)(v / a.Hq) : 0;
      s_row[d] = r;
      s_head[d] = d < nh ? (int)(v - (int64_t)r * a.Hq) : 0;
      // partials of row r: sparse = slot-major list [p0, p0 + np), dense = index w * rows + r
      s_p0[d] = sparse ? (long long)a.slot_base[r] * a.TPC : (long long)r;
      s_np[d] = d >= nh ? 0 : (sparse ? (a.slot_base[r + 1] - a.slot_base[r]) * a.TPC : a.world);
      s_m[d] = -CUDART_INF_F;
      s_l[d] = 0.f;
    }
    __syncthreads();
    int np = 0;
#pragma unroll
    for (int hh = 0; hh < kCombHeads; ++hh) np = max(np, s_np[hh]);
    auto pidx = [&](int hh, int i) -> int64_t {
      return sparse ? (int64_t)s_p0[hh] + i : (int64_t)i * a.rows + s_p0[hh];
    };
    const float* po[kCombHeads];  // this thread's element of partial 0 of each vector
#pragma unroll
    for (int hh = 0; hh < kCombHeads; ++hh)
      po[hh] = a.part_o + ((int64_t)s_p0[hh] * a.Hq + s_head[hh]) * D + d;

    if (np <= kCombFastParts) {
      // ---- every load of the batch in flight at once --------------------------------------------
      float ov[kCombHeads][kCombFastParts];
#pragma unroll
      for (int hh = 0; hh < kCombHeads; ++hh)
#pragma unroll
        for (int i = 0; i < kCombFastParts; ++i)
          ov[hh][i] = i < s_np[hh] ? __ldg(po[hh] + (int64_t)i * pstride) : 0.f;
      if (d < kCombHeads * kCombFastParts) {
        const int i = d / kCombHeads, hh = d - i * kCombHeads;
        const bool valid = i < s_np[hh];
        const int64_t idx = valid ? pidx(hh, i) * a.Hq + s_head[hh] : 0;
        s_w[d] = valid ? __ldg(a.part_m + idx) * mscale : -CUDART_INF_F;              // [i][hh]
        s_w[kCombHeads * kCombFastParts + d] = valid ? (sparse ? __ldg(a.part_l + idx) : 1.f) : 0.f;
      }
      __syncthreads();
      float res[kCombHeads];
#pragma unroll
      for (int hh = 0; hh < kCombHeads; ++hh) {
        float M = -CUDART_INF_F;
#pragma unroll
        for (int i = 0; i < kCombFastParts; ++i) M = fmaxf(M, s_w[i * kCombHeads + hh]);
        const float m_use = M == -CUDART_INF_F ? 0.f : M;
        float L = 0.f, o = 0.f;
#pragma unroll
        for (int i = 0; i < kCombFastParts; ++i) {
          const float w = exp2f(s_w[i * kCombHeads + hh] - m_use);  // 0 for empty partials
          L = fmaf(s_w[kCombHeads * kCombFastParts + i * kCombHeads + hh], w, L);
          o = fmaf(ov[hh][i], w, o);
        }
        res[hh] = (hh < nh && L > 0.f) ? o / L : 0.f;
        if (d == hh && hh < nh && a.lse_out)
          a.lse_out[(int64_t)(s_row[hh] + a.row_offset) * a.Hq + s_head[hh]] =
              L > 0.f ? (M + log2f(L)) * kLn2 : -CUDART_INF_F;
      }
      float4* so4 = reinterpret_cast<float4*>(s_o + d * kCombHeads);  // s_o is [D][8 vectors]
      so4[0] = make_float4(res[0], res[1], res[2], res[3]);
      so4[1] = make_float4(res[4], res[5], res[6], res[7]);
    } else {
      float o[kCombHeads];
#pragma unroll
      for (int hh = 0; hh < kCombHeads; ++hh) o[hh] = 0.f;
      for (int c0 = 0; c0 < np; c0 += kCombMaxParts) {
        const int nc = min(kCombMaxParts, np - c0);
        __syncthreads();
        for (int t = d; t < nc * kCombHeads; t += D) {  // (partial, vector) -> log2-domain maximum
          const int i = t / kCombHeads, hh = t - i * kCombHeads;
          s_w[t] = c0 + i < s_np[hh] ? __ldg(a.part_m + pidx(hh, c0 + i) * a.Hq + s_head[hh]) * mscale
                                     : -CUDART_INF_F;
        }
        __syncthreads();
        if (d < kCombHeads) {  // new running max of vector d; rescale what was accumulated so far
          float M = s_m[d];
          for (int i = 0; i < nc; ++i) M = fmaxf(M, s_w[i * kCombHeads + d]);
          const float m_use = M == -CUDART_INF_F ? 0.f : M;
          const float resc = s_m[d] == -CUDART_INF_F ? 0.f : exp2f(s_m[d] - m_use);
          s_l[d] *= resc;
          s_o[d] = resc;  // s_o[0..7] publishes the rescale factors
          s_m[d] = M;
        }
        __syncthreads();
#pragma unroll
        for (int hh = 0; hh < kCombHeads; ++hh) o[hh] *= s_o[hh];
        __syncthreads();
        for (int t = d; t < nc * kCombHeads; t += D) {
          const int hh = t % kCombHeads;
          const float M = s_m[hh];
          s_w[t] = exp2f(s_w[t] - (M == -CUDART_INF_F ? 0.f : M));  // 0 for empty partials
        }
        __syncthreads();
        if (d < nh) {  // running sum of vector d
          float L = s_l[d];
          for (int i = 0; i < nc; ++i) {
            const float w = s_w[i * kCombHeads + d];
            if (w > 0.f) L = fmaf(sparse ? __ldg(a.part_l + pidx(d, c0 + i) * a.Hq + s_head[d]) : 1.f, w, L);
          }
          s_l[d] = L;
        }
#pragma unroll 8
        for (int i = 0; i < nc; ++i) {  // accumulate: independent loads, eight partials (64 loads) in flight
#pragma unroll
          for (int hh = 0; hh < kCombHeads; ++hh) {
            const float w = s_w[i * kCombHeads + hh];
            if (w > 0.f) o[hh] = fmaf(__ldg(po[hh] + (int64_t)(c0 + i) * pstride), w, o[hh]);
          }
        }
      }
      __syncthreads();
#pragma unroll
      for (int hh = 0; hh < kCombHeads; ++hh) {
        const float L = s_l[hh];
        o[hh] = (hh < nh && L > 0.f) ? o[hh] / L : 0.f;
      }
      float4* so4 = reinterpret_cast<float4*>(s_o + d * kCombHeads);
      so4[0] = make_float4(o[0], o[1], o[2], o[3]);
      so4[1] = make_float4(o[4], o[5], o[6], o[7]);
      if (d < nh && a.lse_out) {
        const float L = s_l[d], M = s_m[d];
        a.lse_out[(int64_t)(s_row[d] + a.row_offset) * a.Hq + s_head[d]] =
            L > 0.f ? (M + log2f(L)) * kLn2 : -CUDART_INF_F;
      }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    float acc[kCombHeads];
    if (a.out_rotated) {
#pragma unroll
      for (int hh = 0; hh < kCombHeads; ++hh) acc[hh] = s_o[d * kCombHeads + hh];
    } else {
#pragma unroll
      for (int hh = 0; hh < kCombHeads; ++hh) acc[hh] = 0.f;
      if (kStagePi) {
#pragma unroll 8
        for (int j = 0; j < D; ++j) {
          const float pv = s_pi[j * D + d];
          const float4 oa = *reinterpret_cast<const float4*>(s_o + j * kCombHeads);
          const float4 ob = *reinterpret_cast<const float4*>(s_o + j * kCombHeads + 4);
          acc[0] = fmaf(oa.x, pv, acc[0]); acc[1] = fmaf(oa.y, pv, acc[1]);
          acc[2] = fmaf(oa.z, pv, acc[2]); acc[3] = fmaf(oa.w, pv, acc[3]);
          acc[4] = fmaf(ob.x, pv, acc[4]); acc[5] = fmaf(ob.y, pv, acc[5]);
          acc[6] = fmaf(ob.z, pv, acc[6]); acc[7] = fmaf(ob.w, pv, acc[7]);
        }
      } else {
        for (int j0 = 0; j0 < D; j0 += 16) {  // column d of Pi from L2, 16 loads in flight
          float pv[16];
#pragma unroll
          for (int u = 0; u < 16; ++u) pv[u] = __ldg(a.rotation + (size_t)(j0 + u) * D + d);
#pragma unroll
          for (int u = 0; u < 16; ++u)
#pragma unroll
            for (int hh = 0; hh < kCombHeads; ++hh)
              acc[hh] = fmaf(s_o[(j0 + u) * kCombHeads + hh], pv[u], acc[hh]);
        }
      }
    }
#pragma unroll
    for (int hh = 0; hh < kCombHeads; ++hh)
      if (hh < nh)
        store_from_float(a.out, a.out_dtype,
                         (int64_t)(s_row[hh] + a.row_offset) * a.out_token_stride +
                             (int64_t)s_head[hh] * a.out_head_stride + d,
                         acc[hh]);
    __syncthreads();  // s_o, s_w and the per-vector entries are rewritten by the next batch
  }
}

template <int D>
int launch_combine_t(const CombineArgs& c, cudaStream_t st, bool pdl) {
  constexpr size_t smem = ((size_t)(D <= 128 ? D * D : 0) + kCombHeads * D +
                           kCombMaxParts * kCombHeads + 2 * kCombHeads) * sizeof(float);
  // (same shared-memory carve-out as the attention kernel it follows: no reconfiguration between them)
  if (!ensure_dynamic_smem<combine_kernel<D>>((int)smem, true)) return TQ4_ERR_CUDA;
  const int64_t n_vec = (int64_t)c.rows * c.Hq;
  int64_t grid = (n_vec + kCombHeads - 1) / kCombHeads;
  if (grid > 3 * (int64_t)sm_count()) grid = 3 * (int64_t)sm_count();
  if (launch_kernel(combine_kernel<D>, dim3((unsigned)grid), dim3(D), smem, st, pdl, c) != cudaSuccess)
    return TQ4_ERR_CUDA;
  TQ4_CHECK_LAUNCH();
  return TQ4_OK;
}

// pdl: the launch follows another kernel of the same entry point (false for the stand-alone merge,
// whose partials come from the caller's preceding kernel or collective)
int launch_combine(const CombineArgs& c, int D, cudaStream_t st, bool pdl) {
  if (c.rows == 0) return TQ4_OK;
  switch (D) {
    case 64: return launch_combine_t<64>(c, st, pdl);
    case 96: return launch_combine_t<96>(c, st, pdl);
    case 128: return launch_combine_t<128>(c, st, pdl);
    case 256: return launch_combine_t<256>(c, st, pdl);
  }
  return TQ4_ERR_UNSUPPORTED;
}

template <int D>
int launch_qrot_plan_t(const AttnArgs& a, cudaStream_t st) {
  using Q = QrotCfg<D>;
  if (!ensure_dynamic_smem<qrot_plan_kernel<D>>((int)Q::smem_bytes, true)) return TQ4_ERR_CUDA;
  const int64_t n_vec = (int64_t)a.sh.rows * a.sh.Hq;
  const unsigned grid = (unsigned)((n_vec + Q::VB - 1) / Q::VB) + 1;
  // (first kernel of an entry point: plain stream-ordered launch, see launch_prologue_t)
  if (launch_kernel(qrot_plan_kernel<D>, dim3(grid), dim3(Q::THREADS), Q::smem_bytes, st, false, a) !=
      cudaSuccess)
    return TQ4_ERR_CUDA;
  TQ4_CHECK_LAUNCH();
  return TQ4_OK;
}

// Prologue of an attention call (a != nullptr) and / or cache write of a few new tokens
// (w != nullptr) in one launch; head_dim 256 (Pi does not fit in shared memory) and large writes
// use the separate kernels.
int launch_prologue(const AttnArgs* a, const CompressArgs* w, int head_dim, cudaStream_t st) {
  if (w && (head_dim > 128 || w->n_tokens * w->num_heads * w->n_sources > kSmallRows)) {
    const int rc = dispatch_compress(*w, head_dim, w->x_dtype, st);
    if (rc != TQ4_OK) return rc;
    w = nullptr;
  }
  if (!a && !w) return TQ4_OK;
  switch (head_dim) {
    case 64: return launch_prologue_t<64>(a, w, st);
    case 96: return launch_prologue_t<96>(a, w, st);
    case 128: return launch_prologue_t<128>(a, w, st);
    case 256: return launch_qrot_plan_t<256>(*a, st);
  }
  return TQ4_ERR_UNSUPPORTED;
}

}  // namespace tq4

// ======================================================================================
// C entry points
// ======================================================================================
extern "C" const char* tq4_version(void) { return "tq4-sm100a 0.1"; }

extern "C" const char* tq4_status_string(int status) {
  switch (status) {
    case TQ4_OK: return "ok";
    case TQ4_ERR_INVALID_ARG: return "invalid argument (null/misaligned pointer or bad size)";
    case TQ4_ERR_UNSUPPORTED: return "unsupported head_dim / head grouping / dtype";
    case TQ4_ERR_CUDA: return "CUDA runtime error at launch";
    case TQ4_ERR_WORKSPACE: return "workspace too small";
    case TQ4_ERR_STATIC_SCRATCH:
      return "request needs more scratch than the built-in static area (TQ4_STATIC_SCRATCH_BYTES); "
             "use tq4_paged_attention with a caller-provided workspace";
  }
  return "unknown status";
}

extern "C" size_t tq4_attention_workspace_bytes(int64_t max_query_rows, int num_q_heads,
                                                int num_kv_heads, int head_dim) {
  tq4::AttnShape sh{};
  if (max_query_rows <= 0 || !tq4::make_shape(sh, num_q_heads, num_kv_heads, head_dim)) return 0;
  const int64_t rows = max_query_rows < tq4::kMaxRowsPerLaunch ? max_query_rows : tq4::kMaxRowsPerLaunch;
  tq4::AttnPlan p;
  const size_t a = tq4::carve_plan(p, nullptr, rows, num_q_heads, head_dim, sh.TPC);
  tq4::make_shape(sh, num_q_heads, num_kv_heads, head_dim, tq4::kMmaWarpsPerCta);
  const size_t b = tq4::carve_plan(p, nullptr, rows, num_q_heads, head_dim, 1, (int64_t)tq4::kMaxSms * sh.TPC);
  return a > b ? a : b;
}

// Shared body of tq4_paged_attention and tq4_write_and_attention: `wr` (optional) is a cache write
// of new tokens that must land before the attention reads the cache.
static int attention_impl(
    const tq4::CompressArgs* wr,
    const void* q, int q_dtype, int64_t num_rows, int num_seqs, int num_q_heads, int num_kv_heads,
    int head_dim, int64_t q_token_stride, int64_t q_head_stride, const uint8_t* cache,
    int64_t cache_block_stride, int64_t cache_token_stride, int64_t num_blocks, int block_size,
    const int32_t* block_table, int64_t bt_stride, const int32_t* seq_lens,
    const int32_t* query_start_loc, const float* k_centroids, int n_k_centroids,
    const float* v_centroids, int n_v_centroids, const float* rotation, float sm_scale, int causal,
    int sliding_window, void* out, int out_dtype, int64_t out_token_stride, int64_t out_head_stride,
    float* lse_out, int out_rotated, void* workspace, size_t workspace_bytes, int mode,
    int* err_flag, void* stream) {
  using namespace tq4;
  if (num_rows < 0 || num_seqs < 0 || block_size <= 0 || num_blocks < 0) return TQ4_ERR_INVALID_ARG;
  if (!supported_head_dim(head_dim)) return TQ4_ERR_UNSUPPORTED;
  if (q_dtype < 0 || q_dtype > 2 || out_dtype < 0 || out_dtype > 2) return TQ4_ERR_UNSUPPORTED;
  if (n_k_centroids <= 0 || n_k_centroids > TQ4_MAX_CENTROIDS || n_v_centroids <= 0 ||
      n_v_centroids > TQ4_MAX_CENTROIDS)
    return TQ4_ERR_UNSUPPORTED;
  AttnArgs a{};
  if (!make_shape(a.sh, num_q_heads, num_kv_heads, head_dim)) return TQ4_ERR_UNSUPPORTED;
  if (num_rows == 0) return wr ? launch_prologue(nullptr, wr, head_dim, (cudaStream_t)stream) : TQ4_OK;
  if (!q || !cache || !block_table || !seq_lens || !k_centroids || !v_centroids || !rotation ||
      !out || !workspace)
    return TQ4_ERR_INVALID_ARG;
  if (((uintptr_t)cache & 3) || (cache_token_stride & 3) || (cache_block_stride & 3) ||
      ((uintptr_t)workspace & 15) ||
      cache_token_stride < row_data_bytes(num_kv_heads, head_dim))
    return TQ4_ERR_INVALID_ARG;
  if (query_start_loc == nullptr && num_rows > num_seqs) return TQ4_ERR_INVALID_ARG;
  const bool mma_ok = attention_mma_supported(a.sh, block_size, cache, cache_block_stride,
                                              cache_token_stride);
  if (mode == 2 && !mma_ok) return TQ4_ERR_UNSUPPORTED;
  if (mode < 0 || mode > 4) return TQ4_ERR_INVALID_ARG;
  const bool use_mma = mode == 2 || mode == 3 || mode == 4 || (mode == 0 && mma_ok);
  if (use_mma)
    make_shape(a.sh, num_q_heads, num_kv_heads, head_dim, mma_warps_per_cta(head_dim, a.sh.GC, num_kv_heads, cache_token_stride));
  const int64_t rows_cap = num_rows < kMaxRowsPerLaunch ? num_rows : kMaxRowsPerLaunch;
  // tensor-core kernel: one partial per (row, span), one span per warp phase of every CTA
  const int part_tpc = use_mma ? 1 : a.sh.TPC;
  const int64_t max_spans = use_mma ? (int64_t)kMaxSms * a.sh.TPC : kMaxCtasPerSlice;
  if (workspace_bytes < carve_plan(a.plan, nullptr, rows_cap, num_q_heads, head_dim, part_tpc, max_spans))
    return TQ4_ERR_WORKSPACE;
  carve_plan(a.plan, workspace, rows_cap, num_q_heads, head_dim, part_tpc, max_spans);

  a.sh.num_seqs = num_seqs;
  a.q = q;
  a.q_dtype = q_dtype;
  a.q_token_stride = q_token_stride;
  a.q_head_stride = q_head_stride;
  a.cache = cache;
  a.cache_block_stride = cache_block_stride;
  a.cache_token_stride = cache_token_stride;
  a.num_blocks = num_blocks;
  a.block_size = block_size;
  a.block_table = block_table;
  a.bt_stride = bt_stride;
  a.seq_lens = seq_lens;
  a.query_start_loc = query_start_loc;
  a.k_centroids = k_centroids;
  a.v_centroids = v_centroids;
  a.n_k_centroids = n_k_centroids;
  a.n_v_centroids = n_v_centroids;
  a.rotation = rotation;
  a.scale_log2e = sm_scale * 1.4426950408889634f;
  a.lut_scale_k = lut_scale(head_dim, n_k_centroids);
  a.lut_scale_v = lut_scale(head_dim, n_v_centroids);
  a.causal = causal;
  a.sliding_window = sliding_window > 0 ? sliding_window : 0;
  a.out = out;
  a.out_dtype = out_dtype;
  a.out_token_stride = out_token_stride;
  a.out_head_stride = out_head_stride;
  a.lse_out = lse_out;
  a.out_rotated = out_rotated;
  a.err_flag = err_flag;

  // chunked prefill (several query rows per sequence) at head_dim 128: tensor-core kernel, one
  // dequantisation of a key tile serves a whole block of query rows
  const bool prefill_ok = prefill_tc_supported(a);
  if ((mode == 3 || mode == 4) && !prefill_ok) return TQ4_ERR_UNSUPPORTED;
  // (automatic only when the query blocks fill the GPU: a CTA owns a (row block, KV head) pair, a
  // small chunk is spread wider by the streaming kernel)
  const int64_t prefill_ctas = (num_rows * a.sh.G / 128) * num_kv_heads;
  const bool use_prefill = mode == 3 || mode == 4 || (mode == 0 && prefill_ok && num_rows >= 8 * (int64_t)num_seqs &&
                                         2 * prefill_ctas >= sm_count());

  const int sms = sm_count();
  int ctas = (use_mma ? 1 : 4) * sms / a.sh.n_slices;
  if (ctas < 1) ctas = 1;
  if (ctas > kMaxCtasPerSlice) ctas = kMaxCtasPerSlice;
  if (use_mma && ctas > kMaxSms) ctas = kMaxSms;
  a.sh.ctas = ctas;
  a.sh.span_ctas = use_mma ? ctas * a.sh.TPC : ctas;
  a.sh.part_tpc = part_tpc;
  cudaStream_t st = (cudaStream_t)stream;
  // Decode calls of up to kFusedMaxRows rows can plan, rotate and write inside the attention kernel
  // (two launches per step) or in a prologue kernel in front of it (three).  Measured on B200, graph
  // replays, head_dim 128, GQA 4: the prologue kernel wins while rows x KV heads <= 512 (8 KV heads:
  // 92.5 against 92.7 us at batch 64 x 4096, 50.1 against 53.4 at batch 16; 4 / 2 / 1 KV heads with
  // batch 128 / 256 / 512: 93.9 against 94.9, 100.5 against 103.0, 123.6 against 132.9 us), the fused
  // form above (8 KV heads: 155.7 against 160.4 us at batch 128, 173.9 against 177.4 at batch 256 x
  // 2048).  TQ4_FUSED_PROLOGUE=1 / 0 forces it.
  int force_fused = -1;
  if (const char* e = getenv("TQ4_FUSED_PROLOGUE")) force_fused = atoi(e) != 0;
  if (getenv("TQ4_NO_FUSED_PROLOGUE") != nullptr) force_fused = 0;
  const bool want_fused = force_fused >= 0 ? force_fused != 0 : num_rows * num_kv_heads > kFusedMinRowHeads;
  a.fused = use_mma && !use_prefill && query_start_loc == nullptr && num_rows <= kFusedMaxRows &&
            head_dim <= 128 && want_fused;

  for (int64_t r0 = 0; r0 < num_rows; r0 += kMaxRowsPerLaunch) {
    a.sh.rows = (int)((num_rows - r0) < kMaxRowsPerLaunch ? (num_rows - r0) : kMaxRowsPerLaunch);
    a.sh.row_offset = (int)r0;
    int rc;
    if (a.fused) {  // no prologue kernel; a decode step's cache write rides in the attention kernel
      a.fused_write = nullptr;
      if (wr && a.sh.NCH == 1 && wr->n_tokens <= num_rows && getenv("TQ4_NO_FUSED_WRITE") == nullptr) {
        a.fused_write = wr;
      } else if (wr) {
        prof_begin(TQ4_PROF_WRITE, st);
        rc = dispatch_compress(*wr, head_dim, wr->x_dtype, st);
        prof_end(TQ4_PROF_WRITE, st);
        if (rc != TQ4_OK) return rc;
      }
    } else {
      prof_begin(TQ4_PROF_PROLOGUE, st);
      rc = launch_prologue(&a, r0 == 0 ? wr : nullptr, head_dim, st);
      prof_end(TQ4_PROF_PROLOGUE, st);
      if (rc != TQ4_OK) return rc;
    }
    prof_begin(TQ4_PROF_ATTENTION, st);
    rc = use_prefill ? launch_prefill_tc(a, st, mode == 4)
                     : (use_mma ? launch_attention_mma(a, st) : launch_attention_fp32(a, st));
    prof_end(TQ4_PROF_ATTENTION, st);
    if (rc != TQ4_OK) return rc;
    CombineArgs c{};
    c.slot_base = use_prefill ? nullptr : a.plan.slot_base;  // prefill: one dense partial per row
    c.world = 1;
    c.TPC = a.sh.part_tpc;
    c.part_o = a.plan.part_o;
    c.part_m = a.plan.part_m;
    c.part_l = a.plan.part_l;
    c.rows = a.sh.rows;
    c.row_offset = a.sh.row_offset;
    c.Hq = num_q_heads;
    c.rotation = rotation;
    c.out = out;
    c.out_dtype = out_dtype;
    c.out_token_stride = out_token_stride;
    c.out_head_stride = out_head_stride;
    c.lse_out = lse_out;
    c.out_rotated = out_rotated;
    prof_begin(TQ4_PROF_COMBINE, st);
    rc = launch_combine(c, head_dim, st, true);
    prof_end(TQ4_PROF_COMBINE, st);
    if (rc != TQ4_OK) return rc;
  }
  return TQ4_OK;
}

extern "C" int tq4_paged_attention(
    const void* q, int q_dtype, int64_t num_rows, int num_seqs, int num_q_heads, int num_kv_heads,
    int head_dim, int64_t q_token_stride, int64_t q_head_stride, const uint8_t* cache,
    int64_t cache_block_stride, int64_t cache_token_stride, int64_t num_blocks, int block_size,
    const int32_t* block_table, int64_t bt_stride, const int32_t* seq_lens,
    const int32_t* query_start_loc, const float* k_centroids, int n_k_centroids,
    const float* v_centroids, int n_v_centroids, const float* rotation, float sm_scale, int causal,
    int sliding_window, void* out, int out_dtype, int64_t out_token_stride, int64_t out_head_stride,
    float* lse_out, int out_rotated, void* workspace, size_t workspace_bytes, int mode,
    int* err_flag, void* stream) {
  return attention_impl(nullptr, q, q_dtype, num_rows, num_seqs, num_q_heads, num_kv_heads, head_dim,
                        q_token_stride, q_head_stride, cache, cache_block_stride, cache_token_stride,
                        num_blocks, block_size, block_table, bt_stride, seq_lens, query_start_loc,
                        k_centroids, n_k_centroids, v_centroids, n_v_centroids, rotation, sm_scale,
                        causal, sliding_window, out, out_dtype, out_token_stride, out_head_stride,
                        lse_out, out_rotated, workspace, workspace_bytes, mode, err_flag, stream);
}

extern "C" int tq4_write_and_attention(
    const void* key, const void* value, int kv_dtype, int64_t n_tokens, int64_t k_token_stride,
    int64_t k_head_stride, int64_t v_token_stride, int64_t v_head_stride,
    const int64_t* slot_mapping, int64_t n_slots, const float* rot_t_even, const float* rot_t_odd,
    const float* k_boundaries, int n_k_boundaries, const float* v_boundaries, int n_v_boundaries,
    const void* q, int q_dtype, int64_t num_rows, int num_seqs, int num_q_heads, int num_kv_heads,
    int head_dim, int64_t q_token_stride, int64_t q_head_stride, uint8_t* cache,
    int64_t cache_block_stride, int64_t cache_token_stride, int64_t num_blocks, int block_size,
    const int32_t* block_table, int64_t bt_stride, const int32_t* seq_lens,
    const int32_t* query_start_loc, const float* k_centroids, int n_k_centroids,
    const float* v_centroids, int n_v_centroids, const float* rotation, float sm_scale, int causal,
    int sliding_window, void* out, int out_dtype, int64_t out_token_stride, int64_t out_head_stride,
    float* lse_out, int out_rotated, void* workspace, size_t workspace_bytes, int mode,
    int* err_flag, void* stream) {
  using namespace tq4;
  if (n_tokens < 0 || n_slots < 0 || num_kv_heads <= 0 || block_size <= 0 || num_blocks < 0)
    return TQ4_ERR_INVALID_ARG;
  if (!supported_head_dim(head_dim) || kv_dtype < 0 || kv_dtype > 2) return TQ4_ERR_UNSUPPORTED;
  if (n_k_boundaries < 0 || n_k_boundaries > TQ4_MAX_BOUNDARIES || n_v_boundaries < 0 ||
      n_v_boundaries > TQ4_MAX_BOUNDARIES)
    return TQ4_ERR_UNSUPPORTED;
  CompressArgs w{};
  const CompressArgs* wr = nullptr;
  if (n_tokens > 0 && n_slots > 0) {
    if (!key || !value || !slot_mapping || !rot_t_even || !rot_t_odd || !k_boundaries || !v_boundaries ||
        !cache)
      return TQ4_ERR_INVALID_ARG;
    if (((uintptr_t)rot_t_even | (uintptr_t)rot_t_odd) & 15) return TQ4_ERR_INVALID_ARG;
    if (((uintptr_t)cache & 3) || (cache_token_stride & 3) ||
        cache_token_stride < row_data_bytes(num_kv_heads, head_dim) ||
        cache_block_stride != (int64_t)block_size * cache_token_stride)  // flat slots = block-major rows
      return TQ4_ERR_INVALID_ARG;
    w.x[0] = key;
    w.x[1] = value;
    w.token_stride[0] = k_token_stride;
    w.head_stride[0] = k_head_stride;
    w.token_stride[1] = v_token_stride;
    w.head_stride[1] = v_head_stride;
    w.bounds[0] = k_boundaries;
    w.n_bounds[0] = n_k_boundaries;
    w.bounds[1] = v_boundaries;
    w.n_bounds[1] = n_v_boundaries;
    w.n_tokens = n_tokens < n_slots ? n_tokens : n_slots;
    w.num_heads = num_kv_heads;
    w.n_sources = 2;
    w.x_dtype = kv_dtype;
    w.rot_even = rot_t_even;
    w.rot_odd = rot_t_odd;
    w.cache = cache;
    w.slot_mapping = slot_mapping;
    w.n_slots = n_slots;
    w.cache_token_stride = cache_token_stride;
    w.num_cache_slots = num_blocks * block_size;
    w.err_flag = err_flag;
    wr = &w;
  }
  return attention_impl(wr, q, q_dtype, num_rows, num_seqs, num_q_heads, num_kv_heads, head_dim,
                        q_token_stride, q_head_stride, cache, cache_block_stride, cache_token_stride,
                        num_blocks, block_size, block_table, bt_stride, seq_lens, query_start_loc,
                        k_centroids, n_k_centroids, v_centroids, n_v_centroids, rotation, sm_scale,
                        causal, sliding_window, out, out_dtype, out_token_stride, out_head_stride,
                        lse_out, out_rotated, workspace, workspace_bytes, mode, err_flag, stream);
}

extern "C" int tq4_combine_partials(const float* parts_o, const float* parts_lse, int world,
                                    int64_t num_rows, int num_q_heads, int head_dim,
                                    const float* rotation, void* out, int out_dtype,
                                    int64_t out_token_stride, int64_t out_head_stride,
                                    void* stream) {
  using namespace tq4;
  if (world <= 0 || num_rows < 0 || num_q_heads <= 0) return TQ4_ERR_INVALID_ARG;
  if (!supported_head_dim(head_dim) || out_dtype < 0 || out_dtype > 2) return TQ4_ERR_UNSUPPORTED;
  if (num_rows == 0) return TQ4_OK;
  if (!parts_o || !parts_lse || !rotation || !out) return TQ4_ERR_INVALID_ARG;
  if (num_rows > 0x7fffffff) return TQ4_ERR_INVALID_ARG;
  CombineArgs c{};
  c.slot_base = nullptr;
  c.world = world;
  c.part_o = parts_o;
  c.part_m = parts_lse;
  c.rows = (int)num_rows;
  c.row_offset = 0;
  c.Hq = num_q_heads;
  c.rotation = rotation;
  c.out = out;
  c.out_dtype = out_dtype;
  c.out_token_stride = out_token_stride;
  c.out_head_stride = out_head_stride;
  return launch_combine(c, head_dim, (cudaStream_t)stream, false);
}

// ======================================================================================
// Allocation-free variant: the scratch lives in the library image.
// ======================================================================================
// One fixed scratch area per GPU that loads the library, held until the process exits.
static __device__ __align__(256) unsigned char g_static_scratch[TQ4_STATIC_SCRATCH_BYTES];

// Device address of g_static_scratch on the CURRENT device.  In host code the symbol's name is
// only a handle, never a device pointer, so the address is asked for once per device with
// cudaGetSymbolAddress (while that device is current) and remembered.
static int static_scratch_address(void** out) {
  static void* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return TQ4_ERR_CUDA;
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr) return TQ4_ERR_CUDA;
    cached[dev] = p;
  }
  *out = cached[dev];
  return TQ4_OK;
}

extern "C" int tq4_paged_attention_static(
    const void* q, int q_dtype, int64_t num_rows, int num_seqs, int num_q_heads, int num_kv_heads,
    int head_dim, int64_t q_token_stride, int64_t q_head_stride, const uint8_t* cache,
    int64_t cache_block_stride, int64_t cache_token_stride, int64_t num_blocks, int block_size,
    const int32_t* block_table, int64_t bt_stride, const int32_t* seq_lens,
    const int32_t* query_start_loc, const float* k_centroids, int n_k_centroids,
    const float* v_centroids, int n_v_centroids, const float* rotation, float sm_scale, int causal,
    int sliding_window, void* out, int out_dtype, int64_t out_token_stride, int64_t out_head_stride,
    int mode, int* err_flag, void* stream) {
  if (num_rows < 0) return TQ4_ERR_INVALID_ARG;
  if (num_rows == 0) return TQ4_OK;
  const size_t need = tq4_attention_workspace_bytes(num_rows, num_q_heads, num_kv_heads, head_dim);
  if (need == 0) return TQ4_ERR_UNSUPPORTED;
  if (need > (size_t)TQ4_STATIC_SCRATCH_BYTES) return TQ4_ERR_STATIC_SCRATCH;
  void* scratch = nullptr;
  const int rc = static_scratch_address(&scratch);
  if (rc != TQ4_OK) return rc;
  return tq4_paged_attention(q, q_dtype, num_rows, num_seqs, num_q_heads, num_kv_heads, head_dim,
                             q_token_stride, q_head_stride, cache, cache_block_stride,
                             cache_token_stride, num_blocks, block_size, block_table, bt_stride,
                             seq_lens, query_start_loc, k_centroids, n_k_centroids, v_centroids,
                             n_v_centroids, rotation, sm_scale, causal, sliding_window, out, out_dtype,
                             out_token_stride, out_head_stride, nullptr, 0, scratch,
                             (size_t)TQ4_STATIC_SCRATCH_BYTES, mode, err_flag, stream);
}
