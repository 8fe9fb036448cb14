/*
 * tq4.h — C ABI of the B200 (sm_100a) TQ4 KV-cache library (libtq4_sm100a.so).
 *
 * TQ4 format (per token, per KV head, per K-or-V): D/2 bytes of nibble-packed 4-bit
 * Lloyd-Max centroid indices (high nibble = even coordinate, low nibble = odd coordinate)
 * followed, in a separate region of the token row, by one little-endian fp32 L2 norm.
 * A paged-cache token row is laid out region-major then head-major:
 *     [K_idx: H*D/2][K_norm: H*4][V_idx: H*D/2][V_norm: H*4][optional padding]
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless stated otherwise; nothing is allocated,
 *     freed or synchronised inside any entry point; work is enqueued on `stream`
 *     (a cudaStream_t passed as void*), so every call is CUDA-graph capturable;
 *   - strides are in ELEMENTS for typed tensors and in BYTES for the uint8 cache;
 *   - every function returns a tq4_status; TQ4_OK means "enqueued";
 *   - `err_flag` (optional, may be NULL) is a device int that kernels OR with a
 *     TQ4_DEV_* bit when they meet an out-of-range slot / block id; the offending access
 *     is skipped, never performed;
 *   - the library keeps no state between calls except per-device lookups it makes once (kernel
 *     attributes, SM count, the address of the built-in scratch), so one process may drive several
 *     GPUs: make the device of the tensors current before a call.  It is thread-compatible (the
 *     caller serialises per stream).
 *
 * Each entry point cites the interface of the reference project (turboquant-vllm v1.5.0,
 * paths relative to its root) that it replaces.
 */
#ifndef TQ4_H_
#define TQ4_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum { TQ4_F32 = 0, TQ4_F16 = 1, TQ4_BF16 = 2 } tq4_dtype;

typedef enum {
  TQ4_OK = 0,
  TQ4_ERR_INVALID_ARG = 1, /* null pointer, negative size, misaligned pointer            */
  TQ4_ERR_UNSUPPORTED = 2, /* head_dim / group size / dtype outside the supported set    */
  TQ4_ERR_CUDA = 3,        /* a CUDA runtime call failed (launch configuration, ...)      */
  TQ4_ERR_WORKSPACE = 4,   /* workspace smaller than tq4_attention_workspace_bytes says  */
  TQ4_ERR_STATIC_SCRATCH = 5 /* request exceeds the built-in scratch of tq4_paged_attention_static */
} tq4_status;

/* bits OR-ed into *err_flag by kernels */
#define TQ4_DEV_BAD_SLOT 1  /* slot_mapping entry >= num_cache_slots            */
#define TQ4_DEV_BAD_BLOCK 2 /* block_table entry outside [0, num_blocks), or a seq_len beyond the
                               bt_stride * block_size tokens a block-table row can address (cut there) */
#define TQ4_DEV_TIMEOUT 4   /* a bounded device-side wait gave up                */
#define TQ4_DEV_WRITE_ORDER 8 /* tq4_write_and_attention: a new token's slot is not the last position of its
                                 sequence; it was written, but this call's attention may not have seen it */

/* Library identification: returns e.g. "tq4-sm100a 0.1". Host call. */
const char* tq4_version(void);
/* Human-readable text for a tq4_status. Host call. */
const char* tq4_status_string(int status);

/*
 * Compress rows:  x[(n,h), 0:D]  ->  packed[(n,h), 0:D/2] (u8), norms[(n,h)] (f32).
 * norm = ||x||_2 (fp32); y = (x / (norm + 1e-10)) * Pi^T; idx = #{b : b < y}; nibble pack.
 * Exactness: given the same rotated coordinates y the bytes are bit-exact (tq4_pack_rotated_rows);
 * end to end a coordinate within ~1e-7 of a boundary may land in the neighbouring bucket, because
 * the rotation's summation order differs from the reference's matmul: at most 1e-4 of the indices
 * (measured 6e-7 on the FFMA kernels, 5e-7 on the tensor-core kernels that take inputs of more
 * than 8192 vectors at head_dim 128; setting TQ4_NO_TC in the environment keeps every input on the
 * FFMA kernels).  Norms are within 3 ulp of a CPU torch.norm and identical across all kernels here.
 * Replaces: tq4_compress() + _tq4_compress_kernel, src/turboquant_vllm/triton/tq4_compress.py:46-148,173-245
 *           (arithmetic contract = its PyTorch path, :248-295 / quantizer.py:112-151).
 * rot_t_even / rot_t_odd: [D, D/2] fp32, the even / odd columns of Pi^T (same split as the
 * reference).  Row (n,h) of x starts at x + n*x_token_stride + h*x_head_stride (elements).
 * head_dim in {64, 96, 128, 256}; n_boundaries <= 15.
 */
int tq4_compress_rows(const void* x, int x_dtype, int64_t n_tokens, int num_heads, int head_dim,
                      int64_t x_token_stride, int64_t x_head_stride,
                      const float* rot_t_even, const float* rot_t_odd,
                      const float* boundaries, int n_boundaries,
                      uint8_t* packed_out, float* norms_out, void* stream);

/*
 * Test hook for the bit-exactness contract: bucketize + nibble-pack rows that are already
 * rotated (fp32 [n_rows, D]).  Same tie rule as torch.bucketize(right=False):
 * idx = #{b : b < y}  (src/turboquant_vllm/lloyd_max.py:208-222).
 */
int tq4_pack_rotated_rows(const float* rotated, int64_t n_rows, int head_dim,
                          const float* boundaries, int n_boundaries,
                          uint8_t* packed_out, void* stream);

/*
 * Cache write: compress K and V of n_tokens new tokens and scatter the packed rows straight
 * into the paged cache in ONE launch.
 * Replaces: TQ4AttentionImpl._compress_and_store, src/turboquant_vllm/vllm/tq4_backend.py:562-624
 *           (two tq4_compress launches + row assembly + index_put).
 * slot_mapping: int64 [n_slots], n_slots <= n_tokens; token i goes to flat slot
 * slot_mapping[i] (= block*block_size + offset); entries < 0 are skipped (padding).
 * cache row s starts at cache + s*cache_token_stride (bytes); only the first
 * H*(D+8) bytes of a row are written.
 */
int tq4_write_paged(const void* key, const void* value, int kv_dtype,
                    int64_t n_tokens, int num_kv_heads, int head_dim,
                    int64_t k_token_stride, int64_t k_head_stride,
                    int64_t v_token_stride, int64_t v_head_stride,
                    const int64_t* slot_mapping, int64_t n_slots,
                    const float* rot_t_even, const float* rot_t_odd,
                    const float* k_boundaries, int n_k_boundaries,
                    const float* v_boundaries, int n_v_boundaries,
                    uint8_t* cache, int64_t cache_token_stride, int64_t num_cache_slots,
                    int* err_flag, void* stream);

/*
 * Decompress rows (rotated space): out[(n,h), 0:D] = centroids[idx] * norm, cast to out_dtype.
 * Replaces: tq4_decompress() + _tq4_decompress_kernel, src/turboquant_vllm/triton/tq4_decompress.py:43-101,126-184.
 */
int tq4_decompress_rows(const uint8_t* packed, const float* norms,
                        const float* centroids, int n_centroids,
                        int64_t n_rows, int head_dim,
                        void* out, int out_dtype, void* stream);

/*
 * Decompress n_slots consecutive token rows of a paged cache into K and V tensors
 * [n_slots, H, D] (rotated space).
 * Replaces: the region slicing + two tq4_decompress calls of TQ4AttentionImpl._decompress_cache,
 *           src/turboquant_vllm/vllm/tq4_backend.py:626-702.
 */
int tq4_decompress_cache(const uint8_t* cache, int64_t cache_token_stride, int64_t n_slots,
                         int num_kv_heads, int head_dim,
                         const float* k_centroids, int n_k_centroids,
                         const float* v_centroids, int n_v_centroids,
                         void* k_out, void* v_out, int out_dtype, void* stream);

/*
 * Scratch size (bytes) for tq4_paged_attention with at most `max_query_rows` query rows.
 * Host call, no CUDA work.
 */
size_t tq4_attention_workspace_bytes(int64_t max_query_rows, int num_q_heads, int num_kv_heads,
                                     int head_dim);

/*
 * Fused paged TQ4 attention over the packed cache.  Rotates the queries by Pi^T, streams the
 * packed K/V pages once, dequantises nibbles through a centroid LUT, fp32 online softmax,
 * accumulates PV in rotated space, merges the split-KV partials and un-rotates by Pi once
 * per head.  Handles decode (query_start_loc == NULL: row i is the single new token of
 * sequence i) and chunked prefill (query_start_loc int32 [num_seqs+1]: sequence i owns query
 * rows [qsl[i], qsl[i+1]); row j of a chunk of length L sits at absolute position
 * seq_len - L + j and, when causal, sees keys <= its position).
 * Replaces: fused_paged_tq4_decode(), src/turboquant_vllm/triton/fused_paged_tq4_attention.py:76-247,255-370
 *           and fused_paged_tq4_int8_prefill(), src/turboquant_vllm/triton/fused_paged_tq4_int8_prefill.py:80-283,291-417
 *           (the latter is single-sequence, prefix-free and INT8; this one is multi-sequence,
 *           prefix-aware and keeps fp32 accumulation).
 *
 * q            [num_rows, Hq, D] (stride in elements), dtype f16 / bf16 / f32
 * cache        u8; block b, token t of the block at b*cache_block_stride + t*cache_token_stride
 * block_table  int32 [num_seqs, >= ceil(seq_len/block_size)], row stride bt_stride (elements)
 * seq_lens     int32 [num_seqs] total KV length of each sequence (already including the new tokens)
 * k_/v_centroids  fp32 LUTs (<= 16 entries each; they differ for asymmetric K4/V3)
 * rotation     fp32 [D, D] (Pi, row-major)
 * sliding_window  0 = unlimited, else a query at position p sees keys in (p - window, p]
 * out          [num_rows, Hq, D], dtype f16 / bf16 / f32 (f32 = parity mode)
 * lse_out      optional fp32 [num_rows, Hq]: natural-log sum-exp of the scaled scores
 *              (-inf for a row that sees no key); with out_rotated != 0 the output stays in
 *              rotated space (normalised) for a later cross-GPU combine.
 * workspace    >= tq4_attention_workspace_bytes(num_rows, Hq, Hkv, D), 16-byte aligned
 * mode         0 = auto, 1 = fp32 CUDA-core kernel, 2 = streaming tensor-core LUT kernel (mma.sync),
 *              3 = chunked-prefill tcgen05 kernel (needs query_start_loc, head_dim 128, 16-byte
 *              aligned K/V regions; TQ4_ERR_UNSUPPORTED otherwise),
 *              4 = the same kernel in its fast form: queries and probabilities enter the tensor
 *              cores as single fp16 terms (mode 3 splits both into hi + lo), which halves the
 *              tensor work and lets their 2^-11 rounding reach the output (about 1e-3 absolute:
 *              at the edge of the 2e-3 parity bound, hence never chosen by mode 0)
 * A row that sees no key (seq_len 0) gets zeros.
 */
int tq4_paged_attention(const void* q, int q_dtype, int64_t num_rows, int num_seqs,
                        int num_q_heads, int num_kv_heads, int head_dim,
                        int64_t q_token_stride, int64_t q_head_stride,
                        const uint8_t* cache, int64_t cache_block_stride, int64_t cache_token_stride,
                        int64_t num_blocks, int block_size,
                        const int32_t* block_table, int64_t bt_stride,
                        const int32_t* seq_lens, const int32_t* query_start_loc,
                        const float* k_centroids, int n_k_centroids,
                        const float* v_centroids, int n_v_centroids,
                        const float* rotation, float sm_scale, int causal, int sliding_window,
                        void* out, int out_dtype, int64_t out_token_stride, int64_t out_head_stride,
                        float* lse_out, int out_rotated,
                        void* workspace, size_t workspace_bytes, int mode,
                        int* err_flag, void* stream);

/*
 * One decode step of a layer: tq4_write_paged of the new tokens followed by tq4_paged_attention,
 * with the cache write folded into the attention's first kernel, so the step costs two or three
 * launches instead of four.  Arguments are the union of the two calls
 * (same meaning and checks); the cache must be block-major contiguous
 * (cache_block_stride == block_size * cache_token_stride), which makes the flat slot
 * s = block * block_size + offset of slot_mapping address row s at cache + s * cache_token_stride.
 * n_tokens == 0 reduces to tq4_paged_attention, num_rows == 0 to tq4_write_paged.
 * Decode calls (query_start_loc == NULL) of up to 512 rows at head_dim <= 128 with more than 512
 * (row, KV head) pairs run as TWO launches (smaller ones too with TQ4_FUSED_PROLOGUE=1 in the
 * environment; =0 turns the form off): the
 * attention kernel plans its tiles, rotates the queries and compresses the new tokens itself, then
 * the merge kernel.  There token i must be the newest token of sequence i, i.e.
 * slot_mapping[i] addresses position seq_lens[i] - 1 through block_table (what a decode step of a
 * serving engine passes): the CTA that reads a sequence's last tile is the one that writes the
 * token into it.  A token whose slot is elsewhere is still written, and TQ4_DEV_WRITE_ORDER is
 * raised because this call's attention may have read that slot before the write; a token of a
 * sequence with seq_lens[i] == 0 must have a negative slot.  Other calls (chunked prefill, more
 * rows, head_dim 256) run the write kernel first, then prologue, attention and merge.
 * Replaces: the body of TQ4AttentionImpl.forward for a decode batch,
 *           src/turboquant_vllm/vllm/tq4_backend.py (_compress_and_store + _fused_decode_path).
 */
int tq4_write_and_attention(const void* key, const void* value, int kv_dtype, int64_t n_tokens,
                            int64_t k_token_stride, int64_t k_head_stride,
                            int64_t v_token_stride, int64_t v_head_stride,
                            const int64_t* slot_mapping, int64_t n_slots,
                            const float* rot_t_even, const float* rot_t_odd,
                            const float* k_boundaries, int n_k_boundaries,
                            const float* v_boundaries, int n_v_boundaries,
                            const void* q, int q_dtype, int64_t num_rows, int num_seqs,
                            int num_q_heads, int num_kv_heads, int head_dim,
                            int64_t q_token_stride, int64_t q_head_stride,
                            uint8_t* cache, int64_t cache_block_stride, int64_t cache_token_stride,
                            int64_t num_blocks, int block_size,
                            const int32_t* block_table, int64_t bt_stride,
                            const int32_t* seq_lens, const int32_t* query_start_loc,
                            const float* k_centroids, int n_k_centroids,
                            const float* v_centroids, int n_v_centroids,
                            const float* rotation, float sm_scale, int causal, int sliding_window,
                            void* out, int out_dtype, int64_t out_token_stride, int64_t out_head_stride,
                            float* lse_out, int out_rotated,
                            void* workspace, size_t workspace_bytes, int mode,
                            int* err_flag, void* stream);

/*
 * Merge `world` per-shard partial results of a sequence-split (split-KV) attention and
 * un-rotate: parts_o fp32 [world, num_rows, Hq, D] (each normalised, rotated space),
 * parts_lse fp32 [world, num_rows, Hq] (natural log; -inf = shard saw no key).
 * out = (sum_w e^{lse_w - M} o_w / sum_w e^{lse_w - M}) * Pi.
 * The reference has no multi-GPU path; this is the consumer of the one NVLink exchange of the
 * long-context variant (partials are gathered into local memory first, e.g. by ncclAllGather).
 */
int tq4_combine_partials(const float* parts_o, const float* parts_lse, int world,
                         int64_t num_rows, int num_q_heads, int head_dim,
                         const float* rotation,
                         void* out, int out_dtype, int64_t out_token_stride, int64_t out_head_stride,
                         void* stream);

/*
 * tq4_paged_attention without any caller-provided (or library-allocated) scratch.
 * No counterpart in the reference.
 *
 * Some callers cannot hand over a workspace because they cannot allocate device memory at the
 * point of the call: a serving engine that has already given every free byte of HBM to the KV
 * cache, a plugin hook that runs after the host framework froze its memory pool, code that must
 * not risk the implicit device synchronisation of cudaMalloc/cudaFree in a latency-critical loop.
 * For them the library carries its own scratch: a fixed array of TQ4_STATIC_SCRATCH_BYTES in the
 * library image (one copy per GPU that loads the library, held until the process exits).
 *
 * Same arguments and results as tq4_paged_attention minus lse_out / out_rotated / workspace.
 *   - Requests whose tq4_attention_workspace_bytes() exceeds TQ4_STATIC_SCRATCH_BYTES return
 *     TQ4_ERR_STATIC_SCRATCH (e.g. 32 query heads, head_dim 128: up to ~270 query rows).
 *   - The entry point calls no cudaMalloc / cudaFree or any allocating routine.  Its FIRST call
 *     on each device looks up the scratch address (cudaGetSymbolAddress, that device current);
 *     make that first call outside of stream capture.
 *   - All calls on a device share the one scratch area.  Nothing in it needs to be zero at entry
 *     (every word a call reads was written earlier by the same call), but two calls whose kernels
 *     overlap on the GPU (different streams) race on it: serialise them.
 */
#define TQ4_STATIC_SCRATCH_BYTES (32u << 20)
int tq4_paged_attention_static(const void* q, int q_dtype, int64_t num_rows, int num_seqs,
                               int num_q_heads, int num_kv_heads, int head_dim,
                               int64_t q_token_stride, int64_t q_head_stride,
                               const uint8_t* cache, int64_t cache_block_stride,
                               int64_t cache_token_stride, int64_t num_blocks, int block_size,
                               const int32_t* block_table, int64_t bt_stride,
                               const int32_t* seq_lens, const int32_t* query_start_loc,
                               const float* k_centroids, int n_k_centroids,
                               const float* v_centroids, int n_v_centroids,
                               const float* rotation, float sm_scale, int causal, int sliding_window,
                               void* out, int out_dtype, int64_t out_token_stride,
                               int64_t out_head_stride, int mode, int* err_flag, void* stream);

/*
 * Per-kernel timing aid (no counterpart in the reference, which times with torch.cuda.Event
 * around whole Python calls, experiments/experiment_020_fused_paged_decode_benchmark.py:232-256).
 * After tq4_profile_start(n) every entry point brackets its kernels with CUDA events recorded
 * on the caller's stream (up to n samples per kind); tq4_profile_read(kind, ms, max) waits for
 * the recorded events and returns the elapsed milliseconds of each sample.  Host calls; not
 * for use during stream capture.
 */
#define TQ4_PROF_WRITE 0     /* fused paged cache write kernel            */
#define TQ4_PROF_PROLOGUE 1  /* query rotation + tile plan kernel         */
#define TQ4_PROF_ATTENTION 2 /* streaming attention kernel (dominant)     */
#define TQ4_PROF_COMBINE 3   /* split merge + un-rotation kernel          */
#define TQ4_PROF_COMPRESS 4  /* contiguous compress-rows kernel           */
#define TQ4_PROF_KINDS 5
int tq4_profile_start(int max_samples);
int tq4_profile_stop(void);
int tq4_profile_read(int kind, float* ms_out, int max_out); /* returns #samples, -1 on error */

#ifdef __cplusplus
}
#endif
#endif /* TQ4_H_ */
