// Tensor-core flash decode: which CTA geometry runs a call, and what both geometries share.
//
// The kernel (flash_mma_impl.cuh) is built twice:
//   w4  : 4 consumer warps + 1 producer per CTA, up to 4 CTAs per SM.  For calls that may overlap their
//         neighbours on the stream (kv_stable and q_stable): many small CTAs of several launches share an
//         SM, so one launch's prologue and hand-over / merge hide behind the others' streaming.
//   w12 : 12 consumer warps + 1 producer, one CTA per SM with a deep ring.  For a call that runs on its
//         own: the whole SM works on it and the ring prefetches most of the chunk while the previous
//         kernel drains.
#include "flash.cuh"

namespace tq {

int launch_flash_mma_w4(const FlashArgs& a, int splits, const MmaOutput& mo, cudaStream_t st);
int launch_flash_mma_w12(const FlashArgs& a, int splits, const MmaOutput& mo, cudaStream_t st);
int flash_mma_ctas_per_sm_w4(const FlashArgs& a);
int flash_mma_ctas_per_sm_w12(const FlashArgs& a);
int flash_mma_resident_ctas_w4();
int flash_mma_resident_ctas_w12();

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
static bool overlapping(const FlashArgs& a) { return a.kv_stable && a.q_stable; }
static int g_last_geometry = 0;   // warps of the geometry launched last (diagnostic)

bool flash_mma_supported(const FlashArgs& a) {
  if (a.dim != 128 || a.rows > 8 || a.mask != nullptr) return false;
  if (a.v_format == TQ_KV_POLAR) {
    if (a.v_bits != 3 && a.v_bits != 4) return false;
    if (!aligned16(a.v_data) || a.v_batch_stride % 4 || a.v_head_stride % 4) return false;
    if (!aligned16(a.v_norms) || a.vn_batch_stride % 4 || a.vn_head_stride % 4) return false;
  } else if (a.v_format == TQ_KV_AFFINE) {
    // 4-bit codes, two groups of 64, with fp16 or 8-bit affine keys (the K8 / V4 configuration)
    if (a.v_bits != 4 || a.v_group != 64) return false;
    if (a.k_format == TQ_KV_POLAR) return false;
    if (!aligned16(a.v_data) || a.v_batch_stride % 16 || a.v_head_stride % 16) return false;
    if (!aligned16(a.v_scales) || !aligned16(a.v_biases) || a.vs_batch_stride % 8 || a.vs_head_stride % 8)
      return false;
  } else {
    return false;
  }
  if (a.k_format == TQ_KV_DENSE) {
    if (a.k_dtype != TQ_F16 && a.k_dtype != TQ_BF16) return false;
    if (!aligned16(a.k_data) || a.k_batch_stride % 8 || a.k_head_stride % 8) return false;
  } else if (a.k_format == TQ_KV_POLAR) {
    if (a.k_bits != 3 && a.k_bits != 4) return false;
    if (!aligned16(a.k_data) || a.k_batch_stride % 4 || a.k_head_stride % 4) return false;
    if (!aligned16(a.k_norms) || a.kn_batch_stride % 4 || a.kn_head_stride % 4) return false;
  } else if (a.k_format == TQ_KV_AFFINE) {
    // 8-bit codes, two groups of 64: one 32-bit word of scales and one of biases per position
    if (a.k_bits != 8 || a.k_group != 64) return false;
    if (!aligned16(a.k_data) || a.k_batch_stride % 16 || a.k_head_stride % 16) return false;
    if (!aligned16(a.k_scales) || !aligned16(a.k_biases) || a.ks_batch_stride % 8 || a.ks_head_stride % 8)
      return false;
  } else {
    return false;
  }
  if (a.new_v != nullptr) {   // in-launch append: dense keys as stored (fp16), or packed keys; packed values
    if (a.v_format != TQ_KV_POLAR || a.k_format == TQ_KV_AFFINE || a.new_k == nullptr) return false;
    if (a.k_format == TQ_KV_DENSE &&
        (a.new_dtype != a.k_dtype || !aligned16(a.new_k) || a.nk_batch_stride % 8 || a.nk_head_stride % 8))
      return false;
  }
  return true;
}


int flash_mma_chunk_multiple() { return 32; }   // split boundaries: keeps every tile start 16-byte aligned
int flash_mma_ctas_per_sm(const FlashArgs& a) {
  return overlapping(a) ? flash_mma_ctas_per_sm_w4(a) : flash_mma_ctas_per_sm_w12(a);
}
int flash_mma_resident_ctas_per_sm() {
  return g_last_geometry == 4 ? flash_mma_resident_ctas_w4() : g_last_geometry == 12 ? flash_mma_resident_ctas_w12() : -1;
}
int64_t flash_mma_header_bytes(int batch, int n_kv_heads) {
  // status block, one split counter per (batch, kv head), eight value-skipping hint words per (batch, kv head)
  return ((16 + (4 + 32) * (int64_t)batch * n_kv_heads) + 15) / 16 * 16;
}
int flash_mma_max_splits() { return 96; }

int launch_flash_mma(const FlashArgs& a, int splits, const MmaOutput& mo, cudaStream_t st) {
  g_last_geometry = overlapping(a) ? 4 : 12;
  return overlapping(a) ? launch_flash_mma_w4(a, splits, mo, st) : launch_flash_mma_w12(a, splits, mo, st);
}

}  // namespace tq
