// Internal argument block shared by the flash-decode kernels and their launcher.
#pragma once

#include "common.cuh"

namespace tq {

struct FlashArgs {
  int batch, n_q_heads, n_kv_heads, n_rep, dim;
  int64_t seq_len, chunk;          // chunk = positions per split
  const int* seq_lens;             // optional per-sequence valid lengths on the device (<= seq_len)

  const void* q;
  int q_dtype, q_prerotated;
  int64_t q_batch_stride, q_head_stride;
  // several query tokens per sequence (the last q_tokens positions, causal): token t of head h is MMA
  // row t * n_rep + (h mod n_rep) of its kv head's group; rows = n_rep * q_tokens <= 8
  int q_tokens, rows;
  int64_t q_token_stride, out_token_stride;

  int k_format, k_bits, k_dtype, k_group;
  const void* k_data;
  int64_t k_batch_stride, k_head_stride;
  const float* k_norms;
  int64_t kn_batch_stride, kn_head_stride;
  const void* k_scales;
  const void* k_biases;
  int64_t ks_batch_stride, ks_head_stride;
  Table16 k_cent;
  SignMask k_signs;

  int v_format, v_bits, v_group;
  int kv_stable;                   // K / V are not written by kernels that may still run when this one starts
  int q_stable;                    // likewise the query and the rows to append
  int ws_exclusive;                // no call that may overlap with this one uses this workspace
  const void* v_data;
  int64_t v_batch_stride, v_head_stride;
  const float* v_norms;
  int64_t vn_batch_stride, vn_head_stride;
  const void* v_scales;
  const void* v_biases;
  int64_t vs_batch_stride, vs_head_stride;
  Table16 v_cent;
  SignMask v_signs;

  float attn_scale;
  float sparse_thr;                // > 0: drop value tiles whose weights are certain to end below it
  int* active_positions;           // optional (batch, n_kv_heads) count of positions accumulated
  const float* mask;
  int64_t mask_batch_stride, mask_head_stride;

  // optional in-launch append of the step's own token (position seq_len - 1): raw rows
  // (batch, n_kv_heads, dim); the CTA that owns the last chunk of a (batch, kv head) group
  // stores / quantizes them into the cache before it streams that chunk
  const void* new_k;
  const void* new_v;
  int new_dtype;
  int64_t nk_batch_stride, nk_head_stride, nv_batch_stride, nv_head_stride;
  Table16 k_thr, v_thr;            // thresholds on the raw butterfly output (make_raw_thresholds)

  // per-split partial state, laid out (splits, batch * n_q_heads[, dim])
  float* part_m;
  float* part_l;
  float* part_acc;
};

int launch_flash_generic(const FlashArgs& a, int splits, cudaStream_t st);

// Tensor-core path (dim 128, n_rep <= 8, fp16 / 3-4-bit packed / 8-bit affine keys,
// 3-4-bit packed or 4-bit affine values, no mask).  flash_mma_supported() says whether
// the arguments qualify; otherwise the caller takes the general kernel.
bool flash_mma_supported(const FlashArgs& a);
int flash_mma_chunk_multiple();
int flash_mma_ctas_per_sm(const FlashArgs& a);   // CTAs of this call's kernel variant that fit on one SM
int flash_mma_resident_ctas_per_sm();   // what the runtime's occupancy query returned (-1: not queried yet)
struct MmaOutput {       // where the tensor-core kernel's fused merge writes
  int* status;           // workspace header word 0
  int* counters;         // one int per (batch, kv head) after the status block, zero between calls
  uint32_t* hints;       // eight words per (batch, kv head) after the counters (value skipping), zero between calls
  int out_mode, out_dtype;
  void* out;
  int64_t out_batch_stride, out_head_stride;
  float* om;
  float* ol;
  float* oacc;
  int n_peers;           // out_mode 1: peers that also receive the merged state (0: none)
  int peer_unordered;    // the peer slots are used by no exchange that may still be in flight
  const float* g_m;      // out_mode 2: this GPU's receive slot (rank 0's block; g_stride floats between ranks)
  const float* g_l;
  const float* g_acc;
  int64_t g_stride;
  uint32_t* g_flags;
  int g_ranks;
  unsigned long long g_limit_ns;
  float* peer_m[8];
  float* peer_l[8];
  float* peer_acc[8];
  uint32_t* peer_counter[8];
};
int64_t flash_mma_header_bytes(int batch, int n_kv_heads);
int flash_mma_max_splits();
int launch_flash_mma(const FlashArgs& a, int splits, const MmaOutput& mo, cudaStream_t st);

// Optional gate of a merge: wait (bounded by a time limit) until `n` flag words have reached `epoch`
// (the parts were pushed by peer GPUs, see exchange.cu); flags == nullptr: no wait.  When the wait
// gives up the status word is set and the merge writes NaN.  With `reset` the block that is last to
// pass the gate sets the flags back to zero (`done` counts the blocks), so the same launch can be
// replayed from a CUDA graph with a constant `epoch` (1: the flags are shared with other merges of a
// slot ring; 2: they are this merge's alone).
struct PeerGate {
  uint32_t* flags;
  int n;
  uint32_t epoch;
  int* status;
  int reset;
  int* done;
  unsigned long long limit_ns;
};
unsigned long long peer_wait_limit_ns();

int launch_merge(const float* pm, int64_t sm, const float* pl, int64_t sl, const float* pacc,
                 int64_t sa, int n_parts, int64_t n_rows,
                 int dim, int rotate, const SignMask& signs, int finalize, void* out, int out_dtype,
                 int64_t out_row_stride, int64_t rows_per_batch, int64_t out_batch_stride,
                 float* om, float* ol, float* oacc, cudaStream_t st, const PeerGate* gate = nullptr);

}  // namespace tq
