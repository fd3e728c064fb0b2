// tq_flash_decode: argument validation, split-K planning, kernel choice, merge.
#include <math.h>
#include <string.h>

#include "common.cuh"
#include "flash.cuh"

namespace tq {

struct Plan {
  int splits;
  int64_t chunk;
  bool mma;
};

static int validate(const tq_flash_params* p) {
  TQ_REQUIRE(p != nullptr, TQ_ERR_BAD_ARG, "params pointer is NULL");
  TQ_REQUIRE(p->struct_bytes == (int32_t)sizeof(tq_flash_params), TQ_ERR_BAD_ARG,
             "struct_bytes %d does not match this library (%zu)", p->struct_bytes,
             sizeof(tq_flash_params));
  TQ_REQUIRE(p->dim >= 32 && p->dim <= 256 && !(p->dim & (p->dim - 1)), TQ_ERR_BAD_DIM,
             "dim must be a power of 2 in [32, 256], got %d", p->dim);
  TQ_REQUIRE(p->batch > 0 && p->n_q_heads > 0 && p->n_kv_heads > 0, TQ_ERR_BAD_ARG,
             "batch and head counts must be positive");
  TQ_REQUIRE(p->n_q_heads % p->n_kv_heads == 0, TQ_ERR_HEAD_MISMATCH,
             "n_q_heads (%d) must equal n_kv_heads (%d) * n_rep", p->n_q_heads, p->n_kv_heads);
  TQ_REQUIRE(p->seq_len > 0, TQ_ERR_BAD_ARG, "seq_len must be positive, got %lld",
             (long long)p->seq_len);
  TQ_REQUIRE(p->q_tokens >= 0 && p->q_tokens <= 8, TQ_ERR_BAD_ARG, "q_tokens must be 0..8, got %d", p->q_tokens);
  if (p->q_tokens > 1) {
    TQ_REQUIRE(p->seq_len >= p->q_tokens, TQ_ERR_BAD_ARG, "seq_len (%lld) counts the q_tokens (%d) new positions",
               (long long)p->seq_len, p->q_tokens);
    TQ_REQUIRE(p->out_mode == 0 && p->n_peers == 0, TQ_ERR_UNSUPPORTED, "several query tokens need out_mode 0");
    TQ_REQUIRE(p->new_k == nullptr && p->new_v == nullptr, TQ_ERR_UNSUPPORTED,
               "the in-launch append takes one token; store a multi-token step's rows before the call");
    TQ_REQUIRE(p->mask == nullptr, TQ_ERR_UNSUPPORTED, "several query tokens are causal; no additive mask");
  }
  TQ_REQUIRE(p->n_peers >= 0 && p->n_peers <= 8, TQ_ERR_BAD_ARG, "n_peers must be 0..8, got %d", p->n_peers);
  TQ_REQUIRE(p->n_peers == 0 || p->out_mode != 0, TQ_ERR_BAD_ARG, "peer targets need out_mode 1 or 2");
  for (int i = 0; i < p->n_peers; ++i)
    TQ_REQUIRE(p->peer_m[i] && p->peer_l[i] && p->peer_acc[i] && p->peer_counter[i] &&
                   (reinterpret_cast<uintptr_t>(p->peer_acc[i]) & 15) == 0,
               TQ_ERR_BAD_ARG, "peer %d: NULL or misaligned target", i);
  TQ_REQUIRE(p->q_dtype >= TQ_F32 && p->q_dtype <= TQ_BF16, TQ_ERR_BAD_ARG, "bad q_dtype");
  switch (p->k_format) {
    case TQ_KV_POLAR:
      TQ_REQUIRE(p->k_bits >= 1 && p->k_bits <= 4, TQ_ERR_BAD_BITS,
                 "Unsupported bit width: %d. Use 1-4.", p->k_bits);
      TQ_REQUIRE(p->k_norms && p->k_centroids_host, TQ_ERR_BAD_ARG, "polar K needs norms and centroids");
      TQ_REQUIRE(p->q_prerotated || p->k_signs_host, TQ_ERR_BAD_ARG, "polar K needs k_signs unless q is pre-rotated");
      break;
    case TQ_KV_DENSE:
      TQ_REQUIRE(p->k_dtype >= TQ_F32 && p->k_dtype <= TQ_BF16, TQ_ERR_BAD_ARG, "bad k_dtype");
      break;
    case TQ_KV_AFFINE:
      TQ_REQUIRE(p->k_bits == 8, TQ_ERR_BAD_BITS, "affine K supports 8-bit codes, got %d", p->k_bits);
      TQ_REQUIRE(p->k_group > 0 && p->dim % p->k_group == 0, TQ_ERR_BAD_ARG, "bad k_group %d", p->k_group);
      TQ_REQUIRE(p->k_scales && p->k_biases, TQ_ERR_BAD_ARG, "affine K needs scales and biases");
      break;
    default: return set_error(TQ_ERR_BAD_ARG, "unknown k_format %d", p->k_format);
  }
  switch (p->v_format) {
    case TQ_KV_POLAR:
      TQ_REQUIRE(p->v_bits >= 1 && p->v_bits <= 4, TQ_ERR_BAD_BITS,
                 "Unsupported bit width: %d. Use 1-4.", p->v_bits);
      TQ_REQUIRE(p->v_norms && p->v_centroids_host && p->v_signs_host, TQ_ERR_BAD_ARG,
                 "polar V needs norms, centroids and signs");
      break;
    case TQ_KV_AFFINE:
      TQ_REQUIRE(p->v_bits == 4 || p->v_bits == 8, TQ_ERR_BAD_BITS,
                 "affine V supports 4- or 8-bit codes, got %d", p->v_bits);
      TQ_REQUIRE(p->v_group > 0 && p->dim % p->v_group == 0, TQ_ERR_BAD_ARG, "bad v_group %d", p->v_group);
      TQ_REQUIRE(p->v_scales && p->v_biases, TQ_ERR_BAD_ARG, "affine V needs scales and biases");
      break;
    default: return set_error(TQ_ERR_BAD_ARG, "unknown v_format %d", p->v_format);
  }
  TQ_REQUIRE(p->q && p->k_data && p->v_data, TQ_ERR_BAD_ARG, "NULL tensor pointer");
  TQ_REQUIRE(p->out_mode >= 0 && p->out_mode <= 2, TQ_ERR_BAD_ARG, "bad out_mode %d", p->out_mode);
  if (p->out_mode != 1)
    TQ_REQUIRE(p->out && p->out_dtype >= TQ_F32 && p->out_dtype <= TQ_BF16, TQ_ERR_BAD_ARG,
               "modes 0 and 2 need out and a valid out_dtype");
  if (p->out_mode == 2) {
    TQ_REQUIRE(p->n_peers > 0, TQ_ERR_BAD_ARG, "mode 2 needs peer targets (its own slot among them)");
    TQ_REQUIRE(p->gather_m && p->gather_l && p->gather_acc && p->gather_flags && p->gather_ranks >= 1 &&
                   p->gather_ranks <= 16,
               TQ_ERR_BAD_ARG, "mode 2 needs the local receive slot, its flag words and 1..16 ranks");
    TQ_REQUIRE((reinterpret_cast<uintptr_t>(p->gather_acc) & 15) == 0 && p->gather_part_stride % 4 == 0,
               TQ_ERR_MISALIGNED, "gather_acc must be 16-byte aligned and gather_part_stride a multiple of 4 floats");
  }
  if (p->out_mode != 0) {
    TQ_REQUIRE(p->part_m && p->part_l && p->part_acc, TQ_ERR_BAD_ARG,
               "mode 1 needs part_m, part_l and part_acc");
    TQ_REQUIRE((reinterpret_cast<uintptr_t>(p->part_acc) & 15) == 0, TQ_ERR_MISALIGNED,
               "part_acc must be 16-byte aligned (its rows are stored as 16-byte vectors)");
  }
  if (p->new_k || p->new_v) {
    TQ_REQUIRE(p->new_k && p->new_v, TQ_ERR_BAD_ARG, "new_k and new_v must be given together");
    TQ_REQUIRE(p->new_dtype >= TQ_F32 && p->new_dtype <= TQ_BF16, TQ_ERR_BAD_ARG, "bad new_dtype");
    TQ_REQUIRE(p->v_format == TQ_KV_POLAR && p->v_boundaries_host, TQ_ERR_UNSUPPORTED,
               "the in-launch append needs packed values and v_boundaries_host");
    TQ_REQUIRE(p->k_format != TQ_KV_AFFINE, TQ_ERR_UNSUPPORTED, "the in-launch append does not cover affine keys");
    TQ_REQUIRE(p->k_format != TQ_KV_POLAR || (p->k_boundaries_host && p->k_signs_host), TQ_ERR_BAD_ARG,
               "appending packed keys needs k_boundaries_host and k_signs_host");
  }
  return TQ_OK;
}

static int fill_args(const tq_flash_params* p, FlashArgs* a) {
  memset(a, 0, sizeof(*a));
  a->batch = p->batch;
  a->n_q_heads = p->n_q_heads;
  a->n_kv_heads = p->n_kv_heads;
  a->n_rep = p->n_q_heads / p->n_kv_heads;
  a->dim = p->dim;
  a->seq_len = p->seq_len;
  a->seq_lens = p->seq_lens_dev;
  a->q = p->q;
  a->q_dtype = p->q_dtype;
  a->q_prerotated = p->q_prerotated;
  a->q_batch_stride = p->q_batch_stride;
  a->q_head_stride = p->q_head_stride;
  a->q_tokens = p->q_tokens > 1 ? p->q_tokens : 1;
  a->rows = a->n_rep * a->q_tokens;
  a->q_token_stride = p->q_token_stride;
  a->out_token_stride = p->out_token_stride;
  a->k_format = p->k_format;
  a->k_bits = (p->k_format == TQ_KV_POLAR || p->k_format == TQ_KV_AFFINE) ? p->k_bits : 4;
  a->k_dtype = p->k_dtype;
  a->k_group = p->k_group > 0 ? p->k_group : p->dim;
  a->k_data = p->k_data;
  a->k_batch_stride = p->k_batch_stride;
  a->k_head_stride = p->k_head_stride;
  a->k_norms = p->k_norms;
  a->kn_batch_stride = p->kn_batch_stride;
  a->kn_head_stride = p->kn_head_stride;
  a->k_scales = p->k_scales;
  a->k_biases = p->k_biases;
  a->ks_batch_stride = p->ks_batch_stride;
  a->ks_head_stride = p->ks_head_stride;
  a->v_format = p->v_format;
  a->v_bits = p->v_bits;
  a->v_group = p->v_group > 0 ? p->v_group : p->dim;
  a->kv_stable = p->kv_stable;
  a->q_stable = p->q_stable;
  a->ws_exclusive = p->workspace_exclusive;
  a->new_k = p->new_k;
  a->new_v = p->new_v;
  a->new_dtype = p->new_dtype;
  a->nk_batch_stride = p->new_k_batch_stride;
  a->nk_head_stride = p->new_k_head_stride;
  a->nv_batch_stride = p->new_v_batch_stride;
  a->nv_head_stride = p->new_v_head_stride;
  a->v_data = p->v_data;
  a->v_batch_stride = p->v_batch_stride;
  a->v_head_stride = p->v_head_stride;
  a->v_norms = p->v_norms;
  a->vn_batch_stride = p->vn_batch_stride;
  a->vn_head_stride = p->vn_head_stride;
  a->v_scales = p->v_scales;
  a->v_biases = p->v_biases;
  a->vs_batch_stride = p->vs_batch_stride;
  a->vs_head_stride = p->vs_head_stride;
  a->attn_scale = p->attn_scale;
  a->sparse_thr = p->sparse_v_threshold > 0.f ? p->sparse_v_threshold : 0.f;
  a->active_positions = p->active_positions;
  a->mask = p->mask;
  a->mask_batch_stride = p->mask_batch_stride;
  a->mask_head_stride = p->mask_head_stride;
  int rc;
  if (p->k_format == TQ_KV_POLAR) {
    for (int i = 0; i < (1 << p->k_bits); ++i) a->k_cent.v[i] = p->k_centroids_host[i];
    if ((!p->q_prerotated || p->new_k) && (rc = make_sign_mask(p->k_signs_host, p->dim, &a->k_signs))) return rc;
    if (p->new_k) make_raw_thresholds(p->k_boundaries_host, (1 << p->k_bits) - 1, p->dim, &a->k_thr);
  }
  if (p->v_format == TQ_KV_POLAR) {
    for (int i = 0; i < (1 << p->v_bits); ++i) a->v_cent.v[i] = p->v_centroids_host[i];
    if ((rc = make_sign_mask(p->v_signs_host, p->dim, &a->v_signs))) return rc;
    if (p->new_v) make_raw_thresholds(p->v_boundaries_host, (1 << p->v_bits) - 1, p->dim, &a->v_thr);
  }
  return TQ_OK;
}

static void make_plan(const tq_flash_params* p, const FlashArgs& a, Plan* plan) {
  plan->mma = flash_mma_supported(a);
  const int mult = plan->mma ? flash_mma_chunk_multiple() : 32;
  const int rgroups = plan->mma ? 1 : (a.n_rep + 7) / 8;
  const int64_t groups = (int64_t)a.batch * a.n_kv_heads * rgroups;
  const int64_t max_splits = (a.seq_len + mult - 1) / mult;
  int64_t splits = p->num_splits;
  if (splits <= 0) {
    const int64_t sms = num_sms();
    int64_t target;
    if (!plan->mma) {
      target = 2 * sms;
    } else if (a.kv_stable && a.q_stable) {
      // A call that may overlap its neighbours on the stream runs as few, long CTAs (half an SM count
      // of them): the CTAs of several launches share every SM (up to four), so prologues, hand-over
      // and merge hide behind the other launches' streaming, and fewer partial states are merged.
      target = sms / 2;
    } else {
      // A call that runs on its own: one CTA per SM.  The CTA that merges a group outlives the others;
      // leaving one SM per group spare for the next launch's CTAs pays off when the chunks barely grow.
      target = sms;
      if ((target - groups) / groups >= 32) target -= groups;
    }
    splits = target / groups;                          // round down: the grid fits one wave
    if (plan->mma && a.kv_stable && a.q_stable) {
      // ... but a long sequence still gets a CTA per 4096 positions: such launches fill the GPU alone
      const int64_t by_work = (a.seq_len + 4095) / 4096;
      if (groups <= target && splits < by_work) splits = by_work;
    }
    if (splits < 1 && plan->mma && a.kv_stable && a.q_stable) {
      // overlapping launches with more groups than the target: the next launch fills the SMs as this
      // one drains, so wave rounding does not matter; two CTAs per group keep each group's tail short
      // without multiplying prologues (measured at 256 groups of 8192 positions: 1 / 2 / 4 splits =
      // 143 / 121 / 123 us)
      splits = a.seq_len >= 4096 ? 2 : 1;
    } else if (splits < 1) {
      // more groups than CTA slots: several waves.  Pick the split count whose CTA count comes
      // closest to a whole number of CTAs per SM (e.g. 256 groups on 148 SMs: 4 splits = 1024
      // CTAs = 6.9 per SM instead of 1.7), keeping at least 1024 positions per CTA.
      splits = 1;
      double best = 1e30;
      for (int64_t s = 1; s <= 8 && (s == 1 || a.seq_len / s >= 1024); ++s) {
        const double per = (double)(groups * s) / (double)sms;
        const double waste = ceil(per) / per;
        if (waste < best - 0.02) {
          best = waste;
          splits = s;
        }
      }
    }
    const int64_t by_len = (a.seq_len + 127) / 128;   // at least 128 positions per split
    if (splits > by_len) splits = by_len;
  }
  if (splits > max_splits) splits = max_splits;
  if (plan->mma && splits > flash_mma_max_splits()) splits = flash_mma_max_splits();
  if (splits < 1) splits = 1;
  int64_t chunk = (a.seq_len + splits - 1) / splits;
  chunk = (chunk + mult - 1) / mult * mult;
  plan->chunk = chunk;
  plan->splits = (int)((a.seq_len + chunk - 1) / chunk);
}

// Workspace layout: [header][acc][m][l].  The header is a
// 16-byte status block (word 0 is set non-zero by a kernel whose bounded wait
// gave up) followed by one split counter per (batch, kv head); the caller
// zero-fills the workspace once when it allocates it and the kernel leaves the
// counters at zero after every call.
static int64_t header_bytes(const tq_flash_params* p, const Plan&) {
  return flash_mma_header_bytes(p->batch, p->n_kv_heads);   // reserved on both paths
}
static int64_t partial_bytes(const tq_flash_params* p, const Plan& plan) {
  if (!plan.mma && p->out_mode == 1 && plan.splits == 1) return 0;
  const int64_t rows = (int64_t)p->batch * p->n_q_heads * (p->q_tokens > 1 ? p->q_tokens : 1);
  const int64_t parts = plan.splits;
  return parts * rows * (p->dim + 2) * (int64_t)sizeof(float);
}
static int64_t workspace_need(const tq_flash_params* p, const Plan& plan) {
  const int64_t part = partial_bytes(p, plan);
  return (plan.mma || part > 0) ? header_bytes(p, plan) + part : 0;
}

}  // namespace tq

using namespace tq;

static thread_local int g_last_kernel = -1;

extern "C" int tq_flash_decode_last_kernel(void) { return g_last_kernel; }
extern "C" int tq_flash_decode_resident_ctas_per_sm(void) { return flash_mma_resident_ctas_per_sm(); }

extern "C" int64_t tq_flash_decode_header_bytes(int batch, int n_kv_heads) {
  if (batch <= 0 || n_kv_heads <= 0) return 0;
  return flash_mma_header_bytes(batch, n_kv_heads);
}

extern "C" int64_t tq_flash_decode_workspace_bytes(const tq_flash_params* p) {
  int rc = validate(p);
  if (rc) return rc;
  FlashArgs a;
  if ((rc = fill_args(p, &a))) return rc;
  Plan plan;
  make_plan(p, a, &plan);
  return workspace_need(p, plan);
}

extern "C" int tq_flash_decode(const tq_flash_params* p) {
  int rc = validate(p);
  if (rc) return rc;
  FlashArgs a;
  if ((rc = fill_args(p, &a))) return rc;
  Plan plan;
  make_plan(p, a, &plan);
  a.chunk = plan.chunk;
  const int64_t need = workspace_need(p, plan);
  TQ_REQUIRE(need == 0 || ((uintptr_t)p->workspace & 15) == 0, TQ_ERR_MISALIGNED,
             "workspace must be 16-byte aligned");
  TQ_REQUIRE(need == 0 || (p->workspace && p->workspace_bytes >= need), TQ_ERR_WORKSPACE,
             "workspace of %lld bytes required, got %lld", (long long)need,
             (long long)p->workspace_bytes);
  const int64_t rows = (int64_t)p->batch * p->n_q_heads * a.q_tokens;
  const bool direct = partial_bytes(p, plan) == 0;
  if (direct) {
    a.part_m = p->part_m;
    a.part_l = p->part_l;
    a.part_acc = p->part_acc;
  } else {
    // [acc][m][l]: the accumulator block stays 16-byte aligned
    float* ws = (float*)((char*)p->workspace + header_bytes(p, plan));
    a.part_acc = ws;
    a.part_m = ws + (int64_t)plan.splits * rows * p->dim;
    a.part_l = a.part_m + (int64_t)plan.splits * rows;
  }
  cudaStream_t st = (cudaStream_t)p->stream;
  g_last_kernel = plan.mma ? 1 : 0;
  if (plan.mma) {   // the kernel's last CTA per (batch, kv head) merges and writes the output
    MmaOutput mo;
    mo.status = (int*)p->workspace;
    mo.counters = (int*)p->workspace + 4;
    mo.hints = (uint32_t*)p->workspace + 4 + (int64_t)p->batch * p->n_kv_heads;
    mo.out_mode = p->out_mode;
    mo.out_dtype = p->out_dtype;
    mo.out = p->out;
    mo.out_batch_stride = p->out_batch_stride;
    mo.out_head_stride = p->out_head_stride;
    mo.om = p->part_m;
    mo.ol = p->part_l;
    mo.oacc = p->part_acc;
    mo.n_peers = p->out_mode != 0 ? p->n_peers : 0;
    mo.g_m = p->gather_m;
    mo.g_l = p->gather_l;
    mo.g_acc = p->gather_acc;
    mo.g_stride = p->gather_part_stride;
    mo.g_flags = p->gather_flags;
    mo.g_ranks = p->gather_ranks;
    mo.g_limit_ns = peer_wait_limit_ns();
    mo.peer_unordered = p->peer_slots_exclusive;
    for (int i = 0; i < 8; ++i) {
      mo.peer_m[i] = p->peer_m[i];
      mo.peer_l[i] = p->peer_l[i];
      mo.peer_acc[i] = p->peer_acc[i];
      mo.peer_counter[i] = p->peer_counter[i];
    }
    return launch_flash_mma(a, plan.splits, mo, st);
  }
  TQ_REQUIRE(p->n_peers == 0, TQ_ERR_UNSUPPORTED, "peer targets need the tensor-core decode path");
  TQ_REQUIRE(a.q_tokens == 1, TQ_ERR_UNSUPPORTED,
             "several query tokens need the tensor-core decode path (dim 128, n_rep * q_tokens <= 8, no mask)");
  TQ_REQUIRE(p->seq_lens_dev == nullptr, TQ_ERR_UNSUPPORTED,
             "device-side sequence lengths (seq_lens_dev) need the tensor-core decode path");
  TQ_REQUIRE(!(p->sparse_v_threshold > 0.f) && p->active_positions == nullptr, TQ_ERR_UNSUPPORTED,
             "value skipping (sparse_v_threshold, active_positions) needs the tensor-core decode path");
  TQ_REQUIRE(p->new_v == nullptr, TQ_ERR_UNSUPPORTED,
             "the in-launch append needs the tensor-core decode path (dim 128, n_rep <= 8, no mask, fp16 or "
             "packed keys, new_k of the keys' type)");
  rc = launch_flash_generic(a, plan.splits, st);
  if (rc) return rc;
  if (direct) return TQ_OK;
  const int rotate = p->v_format == TQ_KV_POLAR;
  return launch_merge(a.part_m, rows, a.part_l, rows, a.part_acc, rows * p->dim, plan.splits, rows, p->dim,
                      rotate, a.v_signs,
                      p->out_mode == 0, p->out, p->out_dtype, p->out_head_stride, p->n_q_heads,
                      p->out_batch_stride, p->part_m, p->part_l, p->part_acc, st);
}
