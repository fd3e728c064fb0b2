// Internal argument block shared by the flash-decode kernels and their launcher.
#pragma once

#include "common.cuh"

namespace tq {

struct FlashArgs {
  int batch, n_q_heads, n_kv_heads, n_rep, dim;
  int64_t seq_len, chunk;          // chunk = positions per split

  const void* q;
  int q_dtype, q_prerotated;
  int64_t q_batch_stride, q_head_stride;

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
  int kv_stable;
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
  const float* mask;
  int64_t mask_batch_stride, mask_head_stride;

  // per-split partial state, laid out (splits, batch * n_q_heads[, dim])
  float* part_m;
  float* part_l;
  float* part_acc;
};

int launch_flash_generic(const FlashArgs& a, int splits, cudaStream_t st);

// Tensor-core path (dim 128, polar or dense keys, polar values, no mask).
// Returns TQ_ERR_UNSUPPORTED without launching when the arguments do not
// qualify; the caller then takes the generic kernel.
bool flash_mma_supported(const FlashArgs& a);
int flash_mma_chunk_multiple();
int flash_mma_ctas_per_sm();
struct MmaOutput {       // where the tensor-core kernel's fused merge writes
  int* status;           // workspace header word 0
  int* counters;         // batch * n_kv_heads ints after the header, zero between calls
  int out_mode, out_dtype;
  void* out;
  int64_t out_batch_stride, out_head_stride;
  float* om;
  float* ol;
  float* oacc;
  float* l1_m;           // level-1 partials: flash_mma_level1_parts() x rows [x dim]
  float* l1_l;
  float* l1_acc;
  int n_peers;           // out_mode 1: peers that also receive the merged state (0: none)
  float* peer_m[8];
  float* peer_l[8];
  float* peer_acc[8];
  uint32_t* peer_counter[8];
};
int64_t flash_mma_header_bytes(int batch, int n_kv_heads);
int flash_mma_max_splits();
int flash_mma_level1_parts();
int launch_flash_mma(const FlashArgs& a, int splits, const MmaOutput& mo, cudaStream_t st);

// Optional gate of a merge: wait (bounded) until `n` flag words have reached `epoch` (the parts
// were pushed by peer GPUs, see exchange.cu); flags == nullptr: no wait.
struct PeerGate {
  const uint32_t* flags;
  int n;
  uint32_t epoch;
  int* status;
};

int launch_merge(const float* pm, int64_t sm, const float* pl, int64_t sl, const float* pacc,
                 int64_t sa, int n_parts, int64_t n_rows,
                 int dim, int rotate, const SignMask& signs, int finalize, void* out, int out_dtype,
                 int64_t out_row_stride, int64_t rows_per_batch, int64_t out_batch_stride,
                 float* om, float* ol, float* oacc, cudaStream_t st, const PeerGate* gate = nullptr);

}  // namespace tq
