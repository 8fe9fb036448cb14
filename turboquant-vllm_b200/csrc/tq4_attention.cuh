// Shared plan / argument structures of the paged TQ4 attention kernels.
//
// Work decomposition (CUDA-graph safe: the grid depends on shapes only, everything that
// depends on seq_lens is computed on the device):
//   * a query ROW r (one query token, all its heads) sees keys [kv_start[r], kv_end[r]);
//   * the keys of a row are cut into 16-token TILES on absolute 16-token boundaries;
//   * all tiles of all rows form one stream, cut into `ctas` equal contiguous SPANS; CTA c
//     works on span c, so load balance is independent of the length distribution;
//   * fp32 kernel: inside a CTA, warp (ts, vh) handles virtual head vh and every TPC-th tile
//     (phase ts); a (row, CTA) intersection is a SEGMENT; every warp writes one partial (m, l, O)
//     per segment into slot slot_base[r] + (c - first_cta(r)), sub-slot ts;
//   * tensor-core kernel: the stream is cut into ctas * TPC spans instead, warp (ts, vh) of CTA c
//     streams span c * TPC + ts for virtual head vh and writes one partial per (row, span) segment;
//   * the combine kernel merges the slots of a row, normalises and un-rotates.
#pragma once
#include "tq4_common.cuh"
#include "tq4_lut_scale.h"

namespace tq4 {

constexpr int kTileTokens = 16;
constexpr int kMaxWarpsPerCta = 8;     // fp32 kernel
constexpr int kMmaWarpsPerCta = 16;    // tensor-core LUT kernel (one CTA per SM)
constexpr int kMaxCtasPerSlice = 148 * 4;  // upper bound used for workspace sizing (fp32 kernel)
constexpr int kMaxSms = 160;               // tensor-core kernel: one CTA per SM, one span per warp phase
constexpr int kMaxRowsPerLaunch = 4096;    // larger query batches are processed in pieces
constexpr int kFusedMaxRows = 512;         // decode calls up to this size plan and rotate inside the attention kernel
// A row is cut into at most this many spans (= partials the merge kernel has to fold for it): a call of
// a few long rows would otherwise hand the merge kernel hundreds of partials per row on a handful of
// CTAs (batch 1 x 8192 tokens: merge 55 us against 16 us for the attention kernel itself).
constexpr int kMaxSpansPerRow = 64;
__host__ __device__ __forceinline__ int tiles_per_span(int total_tiles, int spans, int longest_row_tiles) {
  const int even = (total_tiles + spans - 1) / spans;
  const int capped = (longest_row_tiles + kMaxSpansPerRow - 1) / kMaxSpansPerRow;
  const int t = even > capped ? even : capped;
  return t > 1 ? t : 1;
}
constexpr int kFusedMinRowHeads = 512;     // ... when rows x KV heads exceeds this (else the separate prologue kernel is faster)

struct AttnPlan {
  float* q_rot;      // [rows][Hq][D] fp32, q * Pi^T
  int* kv_start;     // [rows]
  int* kv_end;       // [rows]
  int* row_seq;      // [rows]   block-table row of the sequence that owns the query row
  int* tile_prefix;  // [rows+1] exclusive prefix sum of tiles per row
  int* slot_base;    // [rows+1] exclusive prefix sum of segments per row
  int* scalars;      // [0] total tiles, [1] tiles per span
  float* part_o;     // [slots][TPC][Hq][D]  un-normalised, rotated space
  float* part_m;     // [slots][TPC][Hq]     running max (log2 domain), -inf if empty
  float* part_l;     // [slots][TPC][Hq]     running sum
};

struct AttnShape {
  int rows;       // query rows in this launch
  int row_offset; // index of the first row of this launch within the whole call
  int num_seqs, Hq, Hkv, D, G;  // G = Hq / Hkv
  int GC;         // q heads per virtual head (<= 8)
  int NCH;        // virtual heads per KV head = ceil(G / GC)
  int HPC;        // virtual heads per CTA
  int TPC;        // tile phases per CTA (warps per virtual head)
  int n_slices;   // VH / HPC
  int ctas;       // CTAs per slice
  int span_ctas;  // equal spans the tile stream of a slice is cut into (fp32 kernel: ctas; tensor-core
                  // kernel: ctas * TPC, every warp phase streams its own contiguous span)
  int part_tpc;   // partials per slot (fp32 kernel: TPC, tensor-core kernel: 1)
};

struct AttnArgs {
  AttnPlan plan;
  AttnShape sh;
  const void* q;
  int q_dtype;
  int64_t q_token_stride, q_head_stride;
  const uint8_t* cache;
  int64_t cache_block_stride, cache_token_stride, num_blocks;
  int block_size;
  const int32_t* block_table;
  int64_t bt_stride;
  const int32_t* seq_lens;
  const int32_t* query_start_loc;  // nullptr = decode
  const float* k_centroids;
  const float* v_centroids;
  int n_k_centroids, n_v_centroids;
  const float* rotation;
  float scale_log2e;  // sm_scale * log2(e)
  float lut_scale_k, lut_scale_v;  // fp16 LUT scale factors (tensor-core kernel)
  int causal, sliding_window;
  void* out;
  int out_dtype;
  int64_t out_token_stride, out_head_stride;
  float* lse_out;
  int out_rotated;
  int* err_flag;
  int fused;  // tensor-core kernel: compute the tile plan and rotate the queries inside the kernel
  const CompressArgs* fused_write;  // host side only: the step's cache write, done inside the fused kernel
};

// A sequence cannot be longer than its block-table row (the C interface carries the row stride, not
// the row's width: the stride bounds it).  A longer seq_len is cut there and reported, so no kernel
// reads a page id past the row.
__device__ __forceinline__ int clamp_seq_len(const AttnArgs& a, int len) {
  const long long cap = (long long)a.bt_stride * a.block_size;
  if ((long long)len > cap) {
    if (a.err_flag) atomicOr(a.err_flag, TQ4_DEV_BAD_BLOCK);
    len = (int)cap;
  }
  return len;
}

inline size_t align16(size_t x) { return (x + 15) & ~(size_t)15; }

// Split Hq query heads over warps: a VIRTUAL head is one KV head plus up to 8 of its query
// heads; a CTA holds HPC virtual heads x TPC tile phases = at most 8 warps.
inline bool make_shape(AttnShape& s, int Hq, int Hkv, int D, int max_warps = kMaxWarpsPerCta) {
  if (Hq <= 0 || Hkv <= 0 || Hq % Hkv) return false;
  s.Hq = Hq; s.Hkv = Hkv; s.D = D; s.G = Hq / Hkv;
  s.NCH = (s.G + 7) / 8;
  s.GC = (s.G + s.NCH - 1) / s.NCH;
  const int vh = Hkv * s.NCH;
  s.HPC = 1;
  for (int c = max_warps; c >= 1; --c)
    if (vh % c == 0) { s.HPC = c; break; }
  s.TPC = max_warps / s.HPC;
  s.n_slices = vh / s.HPC;
  return true;
}

// Carve the workspace.  Returns the number of bytes used.
inline size_t carve_plan(AttnPlan& p, void* ws, int64_t rows, int Hq, int D, int TPC,
                         int64_t max_spans = kMaxCtasPerSlice) {
  const int64_t slots = rows + max_spans;
  unsigned char* b = reinterpret_cast<unsigned char*>(ws);
  size_t off = 0;
  auto take = [&](size_t bytes) {
    unsigned char* q = b ? b + off : nullptr;
    off += align16(bytes);
    return q;
  };
  p.q_rot = reinterpret_cast<float*>(take((size_t)rows * Hq * D * 4));
  p.kv_start = reinterpret_cast<int*>(take((size_t)rows * 4));
  p.kv_end = reinterpret_cast<int*>(take((size_t)rows * 4));
  p.row_seq = reinterpret_cast<int*>(take((size_t)rows * 4));
  p.tile_prefix = reinterpret_cast<int*>(take((size_t)(rows + 1) * 4));
  p.slot_base = reinterpret_cast<int*>(take((size_t)(rows + 1) * 4));
  p.scalars = reinterpret_cast<int*>(take(64));
  p.part_o = reinterpret_cast<float*>(take((size_t)slots * TPC * Hq * D * 4));
  p.part_m = reinterpret_cast<float*>(take((size_t)slots * TPC * Hq * 4));
  p.part_l = reinterpret_cast<float*>(take((size_t)slots * TPC * Hq * 4));
  return off;
}

// Launchers implemented in tq4_attention.cu / tq4_decode_mma.cu.
int launch_attention_fp32(const AttnArgs& a, cudaStream_t st);
int launch_attention_mma(const AttnArgs& a, cudaStream_t st);  // returns TQ4_ERR_UNSUPPORTED if shape not covered
// tensor-core (tcgen05) chunked-prefill kernel (tq4_prefill_tc.cu): writes one dense partial per row
// (normalised rotated output in plan.part_o [rows][Hq][D], natural-log LSE in plan.part_m [rows][Hq])
bool prefill_tc_supported(const AttnArgs& a);
int launch_prefill_tc(const AttnArgs& a, cudaStream_t st, bool fast);
int mma_warps_per_cta(int D, int GC, int Hkv, int64_t token_stride = 0);
bool attention_mma_supported(const AttnShape& sh, int block_size, const uint8_t* cache,
                             int64_t block_stride, int64_t token_stride);

}  // namespace tq4
