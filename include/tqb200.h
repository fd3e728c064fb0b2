/*
 * tqb200.h - C ABI of libtqb200.so: the TurboQuant / PolarQuant packed-KV hot
 * path as hand-written sm_100a CUDA kernels.
 *
 * Conventions
 *   - Every function returns 0 (TQ_OK) or a negative tq_status; the message of
 *     the last failure on the calling thread is tq_last_error_string().
 *   - Tensor arguments (vectors, packed words, norms, queries, weights,
 *     outputs, workspace) are DEVICE pointers owned by the caller.  The library
 *     never allocates or frees device memory.
 *   - Codebook-sized parameters (signs[dim], boundaries[2^bits-1],
 *     centroids[2^bits]) are HOST pointers to float32; they are copied into the
 *     kernel's parameter block at launch.  signs must be exactly +1 or -1.
 *   - `stream` is a cudaStream_t passed as void*; launches are asynchronous and
 *     stream-ordered, nothing synchronises.
 *   - Strides are in elements of the pointed-to type unless stated otherwise.
 *   - Packed layout (reference turboquant_mlx/packing.py:16-56): element j of a
 *     vector lives in word j / vpw at bit (j % vpw) * bits, vpw = {1:32, 2:16,
 *     3:10, 4:8}[bits]; a vector of `dim` elements takes ceil(dim / vpw) words.
 *
 * Each entry point cites the reference interface it replaces (path:line inside
 * the reference project).
 */
#ifndef TQB200_H
#define TQB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum tq_status {
  TQ_OK = 0,
  TQ_ERR_BAD_DIM = -1,        /* dim not a power of two or out of range */
  TQ_ERR_BAD_BITS = -2,       /* bits outside 1..4 (8 / 4 for affine) */
  TQ_ERR_HEAD_MISMATCH = -3,  /* n_q_heads != n_kv_heads * n_rep */
  TQ_ERR_MISALIGNED = -4,     /* pointer or stride breaks an alignment rule */
  TQ_ERR_WORKSPACE = -5,      /* workspace missing or too small */
  TQ_ERR_LAUNCH = -6,         /* CUDA reported a launch/runtime error */
  TQ_ERR_BAD_ARG = -7,        /* any other invalid argument */
  TQ_ERR_UNSUPPORTED = -8     /* valid request this build has no kernel for */
} tq_status;

typedef enum tq_dtype { TQ_F32 = 0, TQ_F16 = 1, TQ_BF16 = 2 } tq_dtype;

/* K / V storage formats understood by tq_flash_decode. */
typedef enum tq_kv_format {
  TQ_KV_POLAR = 0,   /* packed PolarQuant words + float32 norms */
  TQ_KV_DENSE = 1,   /* plain fp16 / bf16 / fp32 rows (keys of the V-only cache) */
  TQ_KV_AFFINE = 2   /* group-wise affine codes + fp16 scale / bias per group */
} tq_kv_format;

int tq_version(void);                      /* major * 10000 + minor * 100 + patch */
const char* tq_last_error_string(void);    /* thread-local, never NULL */

/* ---- fused quantize ------------------------------------------------------
 * Replaces fused_quantize (turboquant_mlx/metal.py:147-196) with the rounding
 * of PolarQuantizer.quantize + pack_indices (quantizer.py:75-106,
 * packing.py:26-56): per-vector L2 norm, x / max(norm, 1e-8), sign flip, raw
 * Walsh-Hadamard butterfly, *s then /s with s = float32(1/sqrt(dim)), strict
 * compare with the boundaries, pack.
 * Vector (o, i), o < n_outer, i < n_inner, is read at
 *   x + o * x_outer_stride + i * dim
 * and written at packed + o * packed_outer_stride + i * packed_dim and
 * norms + o * norms_outer_stride + i, so a (B, H, S, D) insert can land
 * directly inside a (B, H, n_alloc, .) cache at a row offset. */
int tq_quantize(const void* x, int x_dtype, int64_t n_outer, int64_t n_inner,
                int64_t x_outer_stride, int dim, int bits,
                const float* signs_host, const float* boundaries_host,
                uint32_t* packed, int64_t packed_outer_stride,
                float* norms, int64_t norms_outer_stride, void* stream);

/* tq_quantize plus, in the same launch, a strided copy of `copy_rows` rows of `copy_row_bytes`
 * bytes (16-byte multiples): the cache append of one step when the keys are stored as they are and
 * the values are PolarQuant-packed (v_only_cache.py:46-60: `KVCache.update_and_fetch` for K, then
 * quantize-on-insert for V).  One launch instead of two in front of every decode attention. */
int tq_quantize_append(const void* x, int x_dtype, int64_t n_outer, int64_t n_inner,
                       int64_t x_outer_stride, int dim, int bits, const float* signs_host,
                       const float* boundaries_host, uint32_t* packed, int64_t packed_outer_stride,
                       float* norms, int64_t norms_outer_stride, const void* copy_src, void* copy_dst,
                       int64_t copy_rows, int64_t copy_row_bytes, int64_t copy_src_stride_bytes,
                       int64_t copy_dst_stride_bytes, void* stream);

/* ---- dequantize ----------------------------------------------------------
 * Replaces dequant_fp16 (metal.py:199-232) and packed_dequantize
 * (kernels.py:123-155): unpack, centroid * s, raw butterfly, * s * signs *
 * norm, cast to out_dtype.  Addressing mirrors tq_quantize. */
int tq_dequantize(const uint32_t* packed, int64_t packed_outer_stride,
                  const float* norms, int64_t norms_outer_stride,
                  int64_t n_outer, int64_t n_inner, int dim, int bits,
                  const float* centroids_host, const float* signs_host,
                  void* out, int out_dtype, int64_t out_outer_stride, void* stream);

/* ---- pre-rotated query ---------------------------------------------------
 * Replaces prerotate_query (metal_kernels_v4.py:119-150):
 * out[h] = raw_butterfly(q[h] * signs), float32, no 1/sqrt(dim). */
int tq_prerotate_query(const void* q, int q_dtype, int64_t n_heads, int64_t q_head_stride,
                       int dim, const float* signs_host, float* out, void* stream);

/* Replaces walsh_hadamard_transform / randomized_hadamard_transform /
 * inverse_randomized_hadamard (rotation.py:7-80) for float32 rows:
 * out = (bfly(x * pre) * s) * post, pre/post optional (NULL = ones). */
int tq_hadamard(const float* x, int64_t n_rows, int dim, const float* pre_signs_host,
                const float* post_signs_host, int normalize, float* out, void* stream);

/* ---- Q.K scores with a pre-rotated query -----------------------------------
 * Replaces prerot_fused_qk_scores (metal_kernels_v4.py:153-221):
 * out[h, p] = (sum_e c[idx[h / n_rep, p, e]] * q_rot[h, e]) * norm[h / n_rep, p] / dim.
 * k_packed head stride in words, k_norms head stride in floats; out is
 * (n_kv * n_rep, seq_len) contiguous float32. */
int tq_prerot_qk_scores(const float* q_rot, const uint32_t* k_packed, int64_t k_head_stride,
                        const float* k_norms, int64_t kn_head_stride, int n_kv_heads,
                        int64_t seq_len, const float* centroids_host, int dim, int bits,
                        int n_rep, float* out, void* stream);

/* Replaces packed_fused_qk_scores (kernels.py:158-196): per-position dequant
 * then dot with the un-rotated query (multi-head only).  Comparator. */
int tq_packed_qk_scores(const float* query, const uint32_t* k_packed, int64_t k_head_stride,
                        const float* k_norms, int64_t kn_head_stride, int n_heads,
                        int64_t seq_len, const float* centroids_host, const float* signs_host,
                        int dim, int bits, float* out, void* stream);

/* ---- weighted V sum, butterfly pulled out ----------------------------------
 * Replaces sparse_v_matvec (sparse_v.py:94-186):
 * out[h] = signs * bfly(sum_{p : w[h,p] >= thr} w[h,p] * norm[p] * c[idx[p]]) / dim,
 * thr = max(threshold, 0).  Needs tq_sparse_v_workspace_bytes() of workspace. */
size_t tq_sparse_v_workspace_bytes(int n_q_heads, int64_t seq_len, int dim);
int tq_sparse_v_matvec(const float* weights, int64_t w_head_stride,
                       const uint32_t* v_packed, int64_t v_head_stride,
                       const float* v_norms, int64_t vn_head_stride, int n_kv_heads,
                       int64_t seq_len, const float* centroids_host, const float* signs_host,
                       int dim, int bits, float threshold, int n_rep, float* out,
                       void* workspace, size_t workspace_bytes, void* stream);

/* No counterpart in the reference.  tq_sparse_v_matvec for callers that cannot
 * hand over a workspace because they cannot allocate device memory themselves
 * (a serving framework that owns all device memory and forbids cudaMalloc in
 * plugin code, a foreign-language binding without an allocator, a decode loop
 * where an allocation would stall the device).  The partial sums go to a fixed
 * array built into the library, tq_sparse_v_noalloc_max_bytes() = 4 MiB per GPU,
 * held by every process that loads the library until it exits; a call that would
 * need more (tq_sparse_v_workspace_bytes() says how much) fails with
 * TQ_ERR_WORKSPACE.  Calls share the array: do not let two of them overlap on
 * the GPU.  The first call on each device looks up the array's address; make
 * that call before any stream capture.  Allocates nothing, ever. */
size_t tq_sparse_v_noalloc_max_bytes(void);
int tq_sparse_v_matvec_noalloc(const float* weights, int64_t w_head_stride,
                               const uint32_t* v_packed, int64_t v_head_stride,
                               const float* v_norms, int64_t vn_head_stride, int n_kv_heads,
                               int64_t seq_len, const float* centroids_host,
                               const float* signs_host, int dim, int bits, float threshold,
                               int n_rep, float* out, void* stream);

/* ---- split-K flash decoding over packed KV ----------------------------------
 * One query token per sequence.  Replaces flash_attention_turboquant
 * (flash_attention.py:168-274) and the composition turboquant_attention
 * (fused_attention.py:20-125) = prerotate_query -> prerot_fused_qk_scores ->
 * scale/mask -> softmax -> sparse_v_matvec, and for dense / affine keys the
 * composition of hybrid_attention.py:45-88, with a batch dimension, split-K
 * over the sequence and grouped-query heads sharing one read of K/V. */
typedef struct tq_flash_params {
  int32_t struct_bytes;        /* sizeof(tq_flash_params) */
  int32_t batch, n_q_heads, n_kv_heads, dim;
  int64_t seq_len;

  const void* q;               /* (batch, n_q_heads, dim) */
  int32_t q_dtype;
  int32_t q_prerotated;        /* 1: q already holds raw_butterfly(q * k_signs) */
  int64_t q_batch_stride, q_head_stride;

  int32_t k_format, k_bits, k_dtype, k_group;   /* k_dtype: dense only; k_group: affine only */
  const void* k_data;          /* polar: uint32 words; dense: elements; affine: uint8 codes */
  int64_t k_batch_stride, k_head_stride;        /* in units of k_data's element type */
  const float* k_norms;        /* polar only */
  int64_t kn_batch_stride, kn_head_stride;
  const void* k_scales;        /* affine only: fp16 (.., seq, dim / group) */
  const void* k_biases;
  int64_t ks_batch_stride, ks_head_stride;
  const float* k_centroids_host;
  const float* k_signs_host;

  int32_t v_format, v_bits, v_group;
  int32_t kv_stable;           /* 1: no K / V row or norm read by this call is written by a kernel that may still
                                  be running when this call's kernel starts (the decode kernel is launched with
                                  programmatic stream serialization: it may start while the kernels in front of
                                  it on the stream drain), so it may fetch K / V at once; 0: wait first */
  const void* v_data;
  int64_t v_batch_stride, v_head_stride;
  const float* v_norms;
  int64_t vn_batch_stride, vn_head_stride;
  const void* v_scales;
  const void* v_biases;
  int64_t vs_batch_stride, vs_head_stride;
  const float* v_centroids_host;
  const float* v_signs_host;

  float attn_scale;
  int32_t num_splits;          /* 0 = choose from the SM count */
  const float* mask;           /* optional additive mask, element [b, h, p] */
  int64_t mask_batch_stride, mask_head_stride;  /* 0 broadcasts */

  void* workspace;             /* tq_flash_decode_workspace_bytes() */
  int64_t workspace_bytes;

  int32_t out_mode;            /* 0: final output; 1: merged partials (m, l, S); 2: partials pushed to the peers,
                                  gathered from them and merged into the final output (see gather_*) */
  int32_t out_dtype;
  void* out;                   /* modes 0 and 2: (batch, n_q_heads, dim) */
  int64_t out_batch_stride, out_head_stride;
  float* part_m;               /* modes 1 and 2: (batch * n_q_heads) */
  float* part_l;               /* modes 1 and 2: (batch * n_q_heads) */
  float* part_acc;             /* modes 1 and 2: (batch * n_q_heads, dim), before the butterfly */
  void* stream;
  /* mode 1, optional (n_peers 0: off; tensor-core path only): the CTA that completes a (batch, kv head)
   * group also stores its rows of the merged state into each peer_m / peer_l / peer_acc [p] (same row
   * layout as part_*; pointers into other GPUs' memory as mapped in this process, or this GPU's own)
   * and then adds 1 to *peer_counter[p] with release semantics at system scope: after
   * batch * n_kv_heads additions all rows are in place (sequence-sharded decode: the push of
   * tq_peer_push done by the decode kernel itself).  No reference counterpart. */
  int32_t n_peers;             /* 0 .. 8 */
  int32_t peer_slots_exclusive; /* 1: no exchange that may still be in flight uses these peer slots (one slot
                                   per layer, say), so a call that waits for nothing (kv_stable, q_stable,
                                   workspace_exclusive) may store into them at once; 0: it first waits for the
                                   launch in front of it (the gated merge that reads a small ring of slots) */
  float* peer_m[8];
  float* peer_l[8];
  float* peer_acc[8];
  uint32_t* peer_counter[8];
  /* 1: the same promise as kv_stable for the query (and new_k / new_v): with both set the kernel
   * reads its inputs without waiting for the launches in front of it and only waits before it
   * first writes the workspace (not even then with workspace_exclusive), so consecutive decode
   * launches overlap (the CTAs of several launches share every SM).  0: wait before reading the query. */
  int32_t q_stable;
  /* Optional in-launch cache append (no reference counterpart; it takes the place of the
   * quantize-on-insert launch of cache.py:131-150 / v_only_cache.py:46-60 in front of a decode
   * step): new_k / new_v are the raw rows (batch, n_kv_heads, dim) of the step's own token.
   * seq_len counts that token; the kernel stores / quantizes the rows into position
   * seq_len - 1 of k_data / v_data (and the norms) and attends over them in the same launch.
   * Tensor-core path only: packed values; keys packed, or dense fp16 with new_dtype TQ_F16.
   * k_boundaries_host / v_boundaries_host: the 2^bits - 1 codebook boundaries. */
  int32_t new_dtype;
  const void* new_k;
  const void* new_v;
  int64_t new_k_batch_stride, new_k_head_stride, new_v_batch_stride, new_v_head_stride;
  const float* k_boundaries_host;
  const float* v_boundaries_host;
  /* Value skipping inside the decode kernel (sparse_v.py:59-65, threshold plumbed at
   * fused_attention.py:109-121).  The reference drops a position from the value sum when its
   * softmax weight is below the threshold.  Here (tensor-core path, > 0 enables) a warp's tile of 16
   * positions is dropped for a (batch, kv head) group when every weight in it is already certain to
   * end below the threshold - weight <= exp(score - running max) / running sum, and weight <=
   * exp(score - largest score the CTA has seen) - so nothing is dropped that the reference would
   * keep, and everything still counts in the softmax sum.  The largest score is shared by all CTAs of
   * a (batch, kv head) group through hint words in the workspace header when the call has its
   * workspace to itself while it runs (workspace_exclusive, or q_stable = 0: it has waited for its
   * predecessor); otherwise a CTA only knows what its own chunk of the sequence has shown so far.
   * active_positions: optional device int32 (batch, n_kv_heads), zeroed by the caller; receives
   * the number of positions whose values were accumulated (count_active_positions semantics per
   * group, sparse_v.py:189-191). */
  float sparse_v_threshold;
  int32_t sparse_reserved;
  int32_t* active_positions;
  /* Optional device array of `batch` int32 (tensor-core path only): the number of valid
   * positions of each sequence, read by the kernel when it runs, at most seq_len (which then is
   * the capacity the launch is planned for).  Serves ragged batches without a mask tensor, and
   * decode loops replayed from a CUDA graph whose lengths advance on the device.  With new_k /
   * new_v the rows go to position seq_lens_dev[b] - 1.  No reference counterpart. */
  const int32_t* seq_lens_dev;
  /* 1: no call that may be in flight together with this one uses this workspace (e.g. one
   * workspace per layer, reused at the next decode step).  With kv_stable and q_stable the kernel
   * then waits for nothing before it finishes its work (only its last CTA waits, at its end, for
   * the preceding launch to complete, so that launches still complete in stream order), and the
   * hand-over and merge of consecutive launches overlap as well.  0: the workspace may be shared
   * with the preceding call on the stream; the kernel waits for that call before writing it. */
  int32_t workspace_exclusive;
  /* out_mode 2 (tensor-core path; no reference counterpart): the all-gather and merge of the
   * sequence-sharded decode inside the decode launch.  As in mode 1 with peers the CTA that
   * completes a (batch, kv head) group stores its merged rows into every rank's receive slot (one of
   * the peer targets is this rank's own slot) and adds 1 to every rank's counter; it then waits -
   * bounded by tq_set_peer_wait_limit_ms - until the gather_ranks counters at gather_flags (this
   * rank's own, one per rank) have each received batch * n_kv_heads additions, merges the ranks' rows
   * found at gather_m / gather_l / gather_acc (rank 0's block of this GPU's slot; rank p's block is
   * gather_part_stride floats further) and writes the final output to `out`.  gather_flags has
   * gather_ranks + 1 zero-initialised words; the kernel leaves them at zero.  A wait that gives up
   * writes 21 + the missing rank to the workspace's status word and NaN to `out`. */
  int32_t gather_ranks;
  const float* gather_m;
  const float* gather_l;
  const float* gather_acc;
  int64_t gather_part_stride;
  uint32_t* gather_flags;
  /* Several query tokens per sequence (tensor-core path, out_mode 0; the reference intercepts
   * single-token steps only, patch.py:19-21, and sends every other step to dense attention over the
   * dequantized cache).  q_tokens in 2..8 with n_rep * q_tokens <= 8: the queries are the LAST
   * q_tokens positions of the sequence, already stored in the cache (seq_len counts them), and
   * attend causally: token t sees positions 0 .. seq_len - q_tokens + t.  q and out gain a token
   * axis with the strides below (in elements); 0 or 1: one token, strides ignored. */
  int32_t q_tokens;
  int32_t q_tokens_reserved;
  int64_t q_token_stride;
  int64_t out_token_stride;
} tq_flash_params;

/* Workspace contract: 16-byte aligned, at least tq_flash_decode_workspace_bytes()
 * bytes.  It starts with a header of tq_flash_decode_header_bytes(batch,
 * n_kv_heads) bytes (a status block, and per (batch, kv head) one split counter and eight
 * value-skipping hint words) that must be zero the first time the workspace is used; every
 * call leaves counters and hint words at zero, so a workspace can be reused by later calls with the same batch * n_kv_heads.
 * Zero the header again before reusing the memory with a different
 * batch * n_kv_heads or after any other use.  Calls on one stream may share a
 * workspace (the kernel orders its workspace accesses after the preceding launch) unless
 * they set workspace_exclusive; calls on different streams must not. */
int64_t tq_flash_decode_header_bytes(int batch, int n_kv_heads);
int64_t tq_flash_decode_workspace_bytes(const tq_flash_params* p);
int tq_flash_decode(const tq_flash_params* p);
/* Which kernel the calling thread's last tq_flash_decode launched: 1 = tensor-core
 * path (dim 128, n_rep <= 8, no mask, 16-byte aligned rows; keys fp16, 3/4-bit packed
 * or 8-bit group-64 affine; values 3/4-bit packed, or 4-bit group-64 affine with fp16
 * or affine keys), 0 = general float32 path, -1 = none yet.  The workspace's first
 * 16 bytes are a status header for the tensor-core path: the caller zero-fills it
 * once; a kernel whose bounded wait gives up writes a non-zero word there (and its
 * output is invalid).  Diagnostic, no reference counterpart. */
int tq_flash_decode_last_kernel(void);
/* CTAs of the tensor-core decode kernel the runtime keeps resident per SM (occupancy query made
 * when a kernel variant is first set up on a device; the design needs 2); -1 before that.
 * Diagnostic, no reference counterpart. */
int tq_flash_decode_resident_ctas_per_sm(void);

/* Merge n_parts partial states (split-K chunks or ranks): part i of row r is at
 * part_m[i * m_part_stride + r], part_l[i * l_part_stride + r] and
 * part_acc[i * acc_part_stride + r * dim ...], so the three fields may be views
 * into one gathered buffer.  m* = max m_i, l* = sum l_i e^(m_i - m*), acc*
 * likewise; out = post(acc*) / l* with post = signs * bfly(.) / dim when
 * v_signs_host is given, identity when NULL; a part with l == 0 is a no-op.
 * No reference counterpart: the reference runs on one device without split-K. */
int tq_merge_partials(const float* part_m, int64_t m_part_stride, const float* part_l,
                      int64_t l_part_stride, const float* part_acc, int64_t acc_part_stride,
                      int n_parts, int64_t n_rows, int dim, const float* v_signs_host,
                      void* out, int out_dtype, int64_t out_row_stride, void* stream);

/* ---- group-wise affine quantisation (K8 / V4) -------------------------------
 * Stands in for KVCache.to_quantized(group_size, bits) as used at
 * hybrid_cache.py:57-63; the arithmetic of the reference lives in the mlx
 * library and is not available, so the format is this library's own:
 * scale = fp16((max - min) / (2^bits - 1)), bias = fp16(min) per group,
 * code = clip(rint((x - bias) / scale), 0, 2^bits - 1); 4-bit codes two per
 * byte, low nibble first. */
int tq_affine_quantize(const void* x, int x_dtype, int64_t n_rows, int dim, int group, int bits,
                       uint8_t* codes, void* scales_f16, void* biases_f16, void* stream);
/* The same with row strides (elements of x; bytes of codes; halfs of scales / biases), so that the
 * rows of one decode step go straight into their places in a pre-sized cache. */
int tq_affine_quantize_rows(const void* x, int x_dtype, int64_t n_rows, int dim, int group, int bits,
                            int64_t x_row_stride, uint8_t* codes, int64_t codes_row_stride,
                            void* scales_f16, void* biases_f16, int64_t sb_row_stride, void* stream);
/* The same with the destination position on the device: the rows go to codes + *position_dev *
 * codes_pos_stride (bytes) and scales / biases + *position_dev * sb_pos_stride (halfs), read when the
 * kernel runs, so that a decode step captured in a CUDA graph appends at a position that advances
 * from replay to replay.  position_dev NULL: as tq_affine_quantize_rows. */
int tq_affine_quantize_rows_at(const void* x, int x_dtype, int64_t n_rows, int dim, int group, int bits,
                               int64_t x_row_stride, uint8_t* codes, int64_t codes_row_stride,
                               void* scales_f16, void* biases_f16, int64_t sb_row_stride,
                               const int32_t* position_dev, int64_t codes_pos_stride, int64_t sb_pos_stride,
                               void* stream);
int tq_affine_dequantize(const uint8_t* codes, const void* scales_f16, const void* biases_f16,
                         int64_t n_rows, int dim, int group, int bits, void* out, int out_dtype,
                         void* stream);

/* Prefill attention over dense 16-bit tensors: out = softmax(scale * Q K^T [+ causal mask]) V
 * for Q (batch, n_q_heads, seq_q, 128), K / V (batch, n_kv_heads, seq_k, 128), all
 * of one dtype (TQ_F16 or TQ_BF16), strides in elements (multiples of 8), 16-byte
 * aligned bases.  With causal != 0 query row i sees keys 0 .. i + (seq_k - seq_q)
 * (seq_k >= seq_q).  Replaces the array-library SDPA the reference falls through to
 * for every call that is not a single-token decode (turboquant_mlx/patch.py:37) on
 * the keys / values returned by update_and_fetch (cache.py:100-150,
 * v_only_cache.py:46-60).  Runs on the tcgen05 tensor cores (accumulators in tensor
 * memory, operands by TMA).  `status` is one zero-initialised device int: a kernel
 * whose bounded wait gives up writes a non-zero code there and returns. */
int tq_prefill_sdpa(const void* q, const void* k, const void* v, void* out, int dtype, int batch,
                    int n_q_heads, int n_kv_heads, int64_t seq_q, int64_t seq_k, int dim,
                    int64_t q_batch_stride, int64_t q_head_stride, int64_t q_row_stride,
                    int64_t k_batch_stride, int64_t k_head_stride, int64_t k_row_stride,
                    int64_t v_batch_stride, int64_t v_head_stride, int64_t v_row_stride,
                    int64_t o_batch_stride, int64_t o_head_stride, int64_t o_row_stride,
                    float attn_scale, int causal, int* status, void* stream);

/* Peer-to-peer exchange of a block between the GPUs of one node (sequence-sharded
 * decode: the per-rank (m, l, acc) partial states that tq_merge_partials combines).
 * tq_peer_push copies `nbytes` from `src` to peer_dst[p] for every p (pointers into the
 * peers' memory as mapped in this process, each the start of the slot that belongs to
 * the calling rank; one of them is the rank's own buffer) and then stores `epoch` to
 * peer_flags[p] with release semantics at system scope.  tq_peer_wait returns, in
 * stream order, once each of the n_ranks 32-bit words at `flags` (this rank's own
 * flag array) has reached `epoch`; its wait is bounded (tq_set_peer_wait_limit_ms), and when it gives
 * up it writes 21 + the missing rank to *status.  The host arrays are read during the call only.
 * No reference counterpart: the reference runs on one device. */
int tq_peer_push(const void* src, int64_t nbytes, void* const* peer_dst, void* const* peer_flags,
                 int n_peers, uint32_t epoch, void* stream);
int tq_peer_wait(const void* flags, int n_ranks, uint32_t epoch, int* status, void* stream);
/* tq_merge_partials whose kernel first performs tq_peer_wait's bounded wait (one launch
 * instead of two): the parts were pushed by the peers with tq_peer_push or by the decode
 * kernel (tq_flash_params.peer_*).  `status` points at two zero-initialised ints: word 0
 * receives 21 + the missing rank when the wait gives up, and the merge then writes NaN
 * instead of a partial result; word 1 is scratch.  With reset_flags != 0 the kernel sets the
 * n_ranks flag words back to zero once all of its blocks are past the wait, so a launch with a
 * constant `epoch` (the additions expected per exchange) can be replayed from a CUDA graph; such
 * a launch also lets the launch behind it on the stream start at once (programmatic dependent
 * launch: the next layer's decode call overlaps this merge and the decode call in front of it).
 * reset_flags 1: the flag words belong to a ring of slots that other merges also wait on, so this
 * merge starts its wait only after the launch in front of it has completed; 2: the flag words are
 * waited on by this merge alone (a slot per layer), it waits for nothing but them, and `flags` has
 * one more zero-initialised word behind the n_ranks flag words (its block count, scratch). */
int tq_merge_partials_after_peers(void* flags, int n_ranks, uint32_t epoch, int* status, int reset_flags,
                                  const float* part_m, int64_t m_part_stride, const float* part_l,
                                  int64_t l_part_stride, const float* part_acc, int64_t acc_part_stride,
                                  int n_parts, int64_t n_rows, int dim, const float* v_signs_host,
                                  void* out, int out_dtype, int64_t out_row_stride, void* stream);
/* Time limit of the peer waits above in milliseconds (default 2000; <= 0 only queries).
 * Returns the previous limit.  The waits stay bounded whatever the value. */
int tq_set_peer_wait_limit_ms(int ms);

#ifdef __cplusplus
}
#endif
#endif /* TQB200_H */
