// Split-K flash decoding for head_dim 128 on tensor cores (sm_100a).
//
// One CTA = one (batch, kv head, sequence chunk).  All n_rep <= 8 query heads of
// the group consume the same K/V bytes, so every KV byte is read once.
//
// The CTA geometry comes from the including file (TQ_FLASH_WARPS consumer warps + 1 producer warp, up to
// TQ_FLASH_MAX_CTAS CTAs per SM): small CTAs, several per SM, for calls whose launches overlap on the
// stream (the CTAs of three to four consecutive launches share every SM, so one launch's prologue, partial-state
// hand-over and merge run while the others stream), one large CTA per SM for a call that runs on its own.
// Every launch is a programmatic dependent launch and releases its successor at entry; what it waits for
// (nothing, when the caller vouches for stable inputs and a workspace of the call's own) is decided per
// argument in the kernel body.
//
//   producer warp : streams tiles of 16 positions per consumer warp of K / V (and their norms) into a
//                   shared-memory ring with cp.async.bulk (TMA, 1-D) and mbarrier
//                   transaction counts; every copy reads this GPU's own memory into
//                   this CTA only.  It also performs the optional in-launch cache
//                   append of the step's own token before it streams the tile that
//                   holds it.
//   consumer warps: each owns 16 positions of a tile and keeps its own online
//                   softmax state, so the main loop has no CTA-wide barrier.
//       scores  : mma.sync m16n8k16 (f16 x f16 -> f32).  A = query rows (rows 0-7
//                 the f16 high part, rows 8-15 the f16 residual, summed after the
//                 MMA, so the query keeps ~22 bits), B = K^T built in registers:
//                 fp16 keys come straight from shared memory; packed keys are
//                 decoded two elements at a time through a lane-replicated pair
//                 LUT in shared memory (conflict-free: entry * 32 + lane); 8-bit
//                 affine codes become f16 (1024 + code) with one PRMT per pair.
//       values  : out^T[e][head] += Vc^T[e][p] * P[p][head]; Vc pairs come from the
//                 same kind of LUT, position pairs are zipped with PRMT.
//       The V norm is folded into the softmax exponent (log2 domain) so P stays
//       <= 2^8 in f16 whatever the norms are; l is accumulated without it.
//   epilogue      : the warps' states are combined through shared memory, the CTA's
//                   (m, l, acc) goes to the workspace (acc in the rotated domain), and
//                   the CTA that completes the (batch, kv head) counter merges all
//                   splits straight from L2 into registers, applies butterfly * signs
//                   / dim / l and writes the output.  No CTA waits for another.
//
// The element <-> MMA k-slot assignment is a free permutation as long as the
// query fragments use the same one; it is chosen per key format so that each
// thread reads contiguous bytes of a row (see kslot_element()).
#include <cuda_fp16.h>

#include <mutex>

#include "flash.cuh"
#include "quantize_row.cuh"

namespace tq {
namespace {

constexpr int kDim = 128;
// CTA geometry, set by the including file: TQ_FLASH_WARPS consumer warps + 1 producer warp per CTA, at
// most TQ_FLASH_MAX_CTAS CTAs per SM (as many as the variant's tables, two stages each and 96 registers
// per thread allow), TQ_GEOM = the suffix of the functions this file exports.
#if !defined(TQ_FLASH_WARPS) || !defined(TQ_FLASH_MAX_CTAS) || !defined(TQ_GEOM)
#error "include this file from a flash_mma_<geometry>.cu that defines TQ_FLASH_WARPS, TQ_FLASH_MAX_CTAS and TQ_GEOM"
#endif
#define TQ_CAT2(a, b) a##b
#define TQ_CAT(a, b) TQ_CAT2(a, b)
constexpr int kConsumerWarps = TQ_FLASH_WARPS;
constexpr int kMaxCtasPerSm = TQ_FLASH_MAX_CTAS;
constexpr int kTile = 16 * kConsumerWarps;   // positions per stage (16 per warp)
constexpr int kChunkMultiple = 32;     // split boundaries: keeps every tile start 16-byte aligned
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kThreads = kConsumerThreads + 32;
constexpr int kMaxStages = 6;
// dynamic shared memory of one CTA when `ctas` of them share an SM (228 KB, 1 KB reserved per CTA, static data)
constexpr int smem_budget(int ctas) { return ctas == 4 ? 55 * 1024 : ctas == 3 ? 74 * 1024 : ctas == 2 ? 112 * 1024 : 224 * 1024; }
// registers per thread that let `ctas` CTAs of kThreads / 32 warps share an SM: the warps spread over four
// schedulers with 16384 registers each, allocated per warp
constexpr int reg_cap(int ctas) {
  const int warps_per_scheduler = (ctas * (kThreads / 32) + 3) / 4;
  const int per_thread = 16384 / warps_per_scheduler / 32 / 8 * 8;
  return per_thread > 128 ? 128 : per_thread;
}
constexpr int kDenseRowBytes = 256;    // rows as in memory: one bulk copy per tile (2-way LDS.128 conflicts accepted)
constexpr uint32_t kSpinLimit = 1u << 22;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.0f;   // log2 units; P stays <= 2^8
constexpr int kMaxParts = 96;               // splits of one (batch, kv head) group
constexpr int kMergeBatch = 12;             // 16-byte loads a merging lane keeps in flight

enum : int { KF_DENSE = 0, KF_DENSE_BF16 = 1, KF_POLAR3 = 3, KF_POLAR4 = 4, KF_AFFINE8 = 8 };
// dense keys: fp16 rows (KF_DENSE) or bf16 rows (KF_DENSE_BF16, scores by the bf16 MMA)
__host__ __device__ constexpr bool is_dense(int kf) { return kf == KF_DENSE || kf == KF_DENSE_BF16; }

struct MmaTables {
  uint16_t k_c16[16];   // beta_k-scaled centroids as f16 bits
  uint16_t v_c16[16];
  float k_post;         // multiplies the raw MMA score: attn_scale * log2(e) [/ (dim * beta_k)]
  float v_post;         // multiplies the accumulator when it is written: 1 / beta_v
  int* status;          // set non-zero if a bounded wait gives up
  int* counters;        // one per (batch, kv head); zero between calls
  uint32_t* hints;      // value skipping: 8 words per (batch, kv head), the largest score any CTA of the group has
                        // seen per head as a biased ordered key (0 = none yet); zero between calls
  int splits;           // partials per (batch, kv head)
  int out_mode, out_dtype;
  void* out;
  int64_t out_batch_stride, out_head_stride;
  float* om;            // merged partial outputs (out_mode 1)
  float* ol;
  float* oacc;
  int n_peers;          // out_mode 1: the merged state also goes to these peers (other GPUs' memory)
  int peer_unordered;   // the peer slots are not shared with an exchange that may still be in flight
  // out_mode 2: after the push the CTA waits (bounded) for every rank's rows of this exchange in this
  // GPU's own receive slot, merges them and writes the final output: the all-gather + merge of the
  // sequence-sharded decode inside the decode launch
  const float* g_m;     // rank 0's block of the local slot; rank p's block is g_stride floats further
  const float* g_l;
  const float* g_acc;
  int64_t g_stride;
  uint32_t* g_flags;    // [n_ranks] counters the ranks' pushes add to, then one word counting this rank's CTAs past the wait
  int g_ranks;
  int g_expect;         // additions per rank and exchange = batch * n_kv_heads
  unsigned long long g_limit_ns;
  float* peer_m[8];
  float* peer_l[8];
  float* peer_acc[8];
  uint32_t* peer_counter[8];
};

template <int KF> struct KGeom;
template <> struct KGeom<KF_DENSE> { static constexpr int row = kDenseRowBytes, lut = 0, norms = 0; };
template <> struct KGeom<KF_DENSE_BF16> { static constexpr int row = kDenseRowBytes, lut = 0, norms = 0; };
template <> struct KGeom<KF_POLAR3> { static constexpr int row = 52, lut = 64 * 32 * 4, norms = kTile * 4; };
// 4-bit keys: the 256-entry pair table is kept once per kK4Rep lanes (lane l reads copy l mod kK4Rep).  One
// copy per lane (32 KB) is conflict free and leaves room for 3 CTAs per SM; 16 copies (16 KB, ~2 wavefronts
// per lookup) let a 4th CTA in and measured 3 % slower on the batch-32 packed-key shape (113.0 vs 109.4 us).
constexpr int kK4Rep = 32;
template <> struct KGeom<KF_POLAR4> { static constexpr int row = 64, lut = 256 * kK4Rep * 4, norms = kTile * 4; };
// group-affine 8-bit codes, two groups of 64: per row 128 code bytes; the "norms" slot holds the
// row's two fp16 scales (4 B) followed, kTile * 4 bytes later, by its two fp16 biases
template <> struct KGeom<KF_AFFINE8> { static constexpr int row = 128, lut = 0, norms = 2 * kTile * 4; };
template <int VB> struct VGeom;
template <> struct VGeom<3> { static constexpr int row = 52, lut = 64 * 32 * 4; };
template <> struct VGeom<4> { static constexpr int row = 64, lut = 256 * 32 * 4; };
// VB == 40: group-affine 4-bit values (two codes per byte, low nibble first: the same bit layout as the
// packed 4-bit rows), groups of 64 elements, one fp16 scale and bias per group and position.
template <> struct VGeom<40> { static constexpr int row = 64, lut = 256 * 32 * 4; };

template <int KF, int VB> struct Layout {
  static constexpr int bars = 0;                         // 2 * stages * 8 bytes (128 reserved)
  static constexpr int q = 128;                          // 16 rows x 128 halfs
  static constexpr int klut = q + 16 * kDim * 2;
  static constexpr int vlut = klut + KGeom<KF>::lut;
  static constexpr int stage0 = vlut + VGeom<VB>::lut;
  static constexpr int k_off = 0;
  static constexpr int kn_off = kTile * KGeom<KF>::row;
  static constexpr int v_off = kn_off + KGeom<KF>::norms;
  static constexpr int vn_off = v_off + kTile * VGeom<VB>::row;
  static constexpr int stage_bytes = vn_off + kTile * (VB == 40 ? 8 : 4);   // norms, or scale + bias words
  // CTAs per SM: as many (up to kMaxCtasPerSm) as still leave two stages each and at least 96 registers per thread
  static constexpr bool fits4 = kMaxCtasPerSm >= 4 && stage0 + 2 * stage_bytes <= smem_budget(4) && reg_cap(4) >= 96;
  static constexpr bool fits3 = kMaxCtasPerSm >= 3 && stage0 + 2 * stage_bytes <= smem_budget(3) && reg_cap(3) >= 96;
  static constexpr bool fits2 = kMaxCtasPerSm >= 2 && stage0 + 2 * stage_bytes <= smem_budget(2) && reg_cap(2) >= 96;
  static constexpr int ctas = fits4 ? 4 : fits3 ? 3 : fits2 ? 2 : 1;
  static constexpr int max_regs = reg_cap(ctas);
  static constexpr int budget = smem_budget(ctas);
  static constexpr int fit = (budget - stage0) / stage_bytes;
  static constexpr int stages = fit > kMaxStages ? kMaxStages : fit;
  // the ring is reused by the epilogue: warp exchange, then the merge's scratch
  static constexpr int xch_rows = VB == 40 ? 36 : 34;   // 32 accumulator values, m, l [, two bias sums]
  static constexpr int xch_bytes = kConsumerWarps * xch_rows * 32 * 4;
  static constexpr int merge_bytes = (8 * kMaxParts + 16) * 4;
  static constexpr int ring_bytes = stages * stage_bytes;
  static constexpr int work_bytes =
      ring_bytes > merge_bytes ? (ring_bytes > xch_bytes ? ring_bytes : xch_bytes)
                               : (merge_bytes > xch_bytes ? merge_bytes : xch_bytes);
  static constexpr int total = stage0 + work_bytes;
  static_assert(stages >= 2, "at least two stages must fit");
  static_assert(2 * stages * 8 <= 128, "barrier block");
  static_assert(stage_bytes % 16 == 0 && stage0 % 16 == 0, "stage alignment");
  static_assert(total <= budget, "shared memory per CTA");
};

// ---- PTX wrappers -----------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
// Bounded wait: false when the phase did not complete within the spin limit.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
  }
  return false;
}
// The same for the producer warp, which is usually a whole ring ahead of the consumers: it polls at a
// low rate, so that its polling takes no issue slots from the warps that do the work.
__device__ __forceinline__ bool mbar_wait_relaxed(uint32_t bar, uint32_t parity) {
  for (uint32_t it = 0; it < kSpinLimit; ++it) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    if (done) return true;
    __nanosleep(256);
  }
  return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
      "l"(src), "r"(bytes), "r"(bar)
      : "memory");
}
__device__ __forceinline__ void consumer_barrier() {
  asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}
__device__ __forceinline__ void grid_dependency_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
}
__device__ __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma16816_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
      "{%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// a pair of floats as the score MMA's 16-bit operand type (high part) and what is left (residual)
template <bool BF>
__device__ __forceinline__ void split_pair(float x, float y, uint32_t& hi, uint32_t& lo) {
  if (BF) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(x, y);
    const float2 hf = __bfloat1622float2(h);
    const __nv_bfloat162 l = __floats2bfloat162_rn(x - hf.x, y - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
  } else {
    const __half2 h = __floats2half2_rn(x, y);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(x - hf.x, y - hf.y);
    hi = *reinterpret_cast<const uint32_t*>(&h);
    lo = *reinterpret_cast<const uint32_t*>(&l);
  }
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float lg2(float x) {
  float y;
  asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
  return v;
}
// Table lookups go through the shared array itself, so that the table's offset inside the shared window
// becomes the load's immediate instead of an add per lookup.
__device__ __forceinline__ uint32_t lut_ld(const uint8_t* table, uint32_t byte_off) {
  return *reinterpret_cast<const uint32_t*>(table + byte_off);
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
  return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
  return v;
}
__device__ __forceinline__ float lds_f32(uint32_t addr) { return __uint_as_float(lds32(addr)); }
__device__ __forceinline__ uint32_t hmul2_bits(uint32_t a, uint32_t b) {
  const __half2 r = __hmul2(*reinterpret_cast<const __half2*>(&a), *reinterpret_cast<const __half2*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t pack_h2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Element of the head dimension that MMA k-step `ks`, k-slot `s` (0..15) stands
// for, per key format.  Slots (2t, 2t+1) and (2t+8, 2t+9) belong to thread t of a
// quad; the two slots of a pair are consecutive elements.
template <int KF>
__device__ __forceinline__ int kslot_element(int ks, int s) {
  const int tt = (s & 7) >> 1, lo = s & 1, up = s >> 3;
  if (is_dense(KF)) return 8 * (4 * (ks >> 1) + tt) + 4 * (ks & 1) + 2 * up + lo;
  if (KF == KF_POLAR4) return 32 * tt + 4 * ks + 2 * up + lo;
  if (KF == KF_AFFINE8) return 16 * (4 * (ks >> 2) + tt) + 4 * (ks & 3) + 2 * up + lo;   // k-steps 0-3: group 0
  const int pi = 2 * ks + up;   // pair index within the thread: 15 pairs in words 3t..3t+2, one in word 12
  return (pi < 15 ? 30 * tt + 2 * pi : 120 + 2 * tt) + lo;
}

// float <-> int with the same ordering (for atomicMax on shared memory); an involution
__device__ __forceinline__ int ordered_int(float f) {
  const int i = __float_as_int(f);
  return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float from_ordered_int(int i) { return __int_as_float(i ^ ((i >> 31) & 0x7fffffff)); }

template <typename T>
__device__ __forceinline__ float load_q(const void* base, int64_t idx) {
  return to_f32<T>(reinterpret_cast<const T*>(base)[idx]);
}
__device__ __forceinline__ float load_any(const void* base, int dtype, int64_t idx) {
  return dtype == TQ_F32 ? load_q<float>(base, idx)
         : dtype == TQ_F16 ? load_q<__half>(base, idx)
                           : load_q<__nv_bfloat16>(base, idx);
}

// One row of the merged result, held by one warp (lane = elements 4*lane .. 4*lane+3):
// final output (butterfly * signs / dim / l) or the merged partial state, which may also
// go to peer GPUs by plain stores.
template <bool VAFF>
__device__ __forceinline__ void write_row(const FlashArgs& a, const MmaTables& tb, int b, int h0, int r, int64_t row,
                                          float4 acc4, float m_star, float l_star, int lane, bool final_out) {
  if (!final_out) {
    reinterpret_cast<float4*>(tb.oacc + row * kDim)[lane] = acc4;
    if (lane == 0) {
      tb.om[row] = m_star;
      tb.ol[row] = l_star;
    }
#pragma unroll
    for (int p = 0; p < 8; ++p) {               // plain peer stores over NVLink (static indices: no local copy)
      if (p < tb.n_peers) {
        reinterpret_cast<float4*>(tb.peer_acc[p] + row * kDim)[lane] = acc4;
        if (lane == 0) {
          tb.peer_m[p][row] = m_star;
          tb.peer_l[p][row] = l_star;
        }
      }
    }
    return;
  }
  float v[4] = {acc4.x, acc4.y, acc4.z, acc4.w};
  if (!VAFF) warp_butterfly<4>(v, lane);      // packed values are summed in the rotated domain
  const float inv = l_star > 0.f ? (VAFF ? 1.0f : 1.0f / kDim) / l_star : 0.f;
  const int tok = r / a.n_rep, head = h0 + r - tok * a.n_rep;   // row r of the group = (query token, head)
  const int64_t ooff = b * tb.out_batch_stride + (int64_t)head * tb.out_head_stride + tok * a.out_token_stride + lane * 4;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float res = v[j] * (VAFF ? 1.0f : sign_at(a.v_signs, lane * 4 + j)) * inv;
    if (tb.out_dtype == TQ_F32) reinterpret_cast<float*>(tb.out)[ooff + j] = res;
    else if (tb.out_dtype == TQ_F16) reinterpret_cast<__half*>(tb.out)[ooff + j] = __float2half_rn(res);
    else reinterpret_cast<__nv_bfloat16*>(tb.out)[ooff + j] = __float2bfloat16_rn(res);
  }
}

// ---- the kernel ---------------------------------------------------------------------
// PLAIN: the call uses none of the per-tile options (value skipping, active-position counts, several
// query tokens); their tests and code are compiled out of the main loop (measured: -2 % on the fp16-key
// shape, -8 % on the packed-key shape).
template <int KF, int VB, bool PLAIN>
__global__ void __maxnreg__((Layout<KF, VB>::max_regs))
flash_mma_kernel(const FlashArgs a, const MmaTables tb) {
  using L = Layout<KF, VB>;
  constexpr int kStages = L::stages;
  extern __shared__ __align__(128) uint8_t smem[];
  const uint32_t sbase = smem_u32(smem);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
  // valid positions of this sequence: the launch's seq_len, or the device-side length when given
  // (an input like the query: unless the caller vouches for it, wait for the preceding grid first)
  if (a.seq_lens != nullptr && !a.q_stable) grid_dependency_wait();
  const int64_t seq = a.seq_lens != nullptr ? max((int64_t)0, min((int64_t)a.seq_lens[b], a.seq_len)) : a.seq_len;
  const int64_t pb = (int64_t)split * a.chunk;
  const int64_t pe = max(pb, min(seq, pb + a.chunk));
  const int n_tiles = (int)((pe - pb + kTile - 1) / kTile);
  const int h0 = kvh * a.n_rep;

  // Programmatic dependent launch: let the next kernel on the stream be scheduled as
  // soon as resources free up; its own griddepcontrol.wait keeps it from consuming
  // anything this grid produces before this grid has completed.
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  auto full_bar = [&](int s) { return sbase + L::bars + 8 * s; };
  auto empty_bar = [&](int s) { return sbase + L::bars + 8 * (kStages + s); };

  __shared__ uint16_t c16_s[32];
  __shared__ float qsum_s[16];     // affine keys: per head and 64-element group, sum of the query
  __shared__ int abort_s;          // a bounded wait of this CTA gave up
  __shared__ int elected_s;        // this CTA completed its group's counter
  __shared__ uint8_t idx_s[kDim];  // producer warp: codes of the row being appended
  __shared__ int hint_s[8];        // value skipping: per head, the largest score any warp of the CTA has seen
  if (tid < 8) hint_s[tid] = (int)0x807FFFFF;   // ordered_int(-inf): decodes to -inf, below every score
  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), kConsumerWarps);
    }
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (tid < 16) c16_s[tid] = tb.v_c16[tid];
  else if (tid < 32) c16_s[tid] = tb.k_c16[tid - 16];
  __syncthreads();   // barriers and codebooks visible; the producer leaves for its loop now
  // pair LUTs: entry (i0 | i1 << bits) replicated per lane -> word index entry * 32 + lane
  if (warp < kConsumerWarps) {
    constexpr int kCT = kConsumerThreads;
    uint32_t* vl = reinterpret_cast<uint32_t*>(smem + L::vlut);
    constexpr int VBITS = VB == 40 ? 4 : VB;
    constexpr int nv = 1 << (2 * VBITS);
    for (int i = tid; i < nv * 32; i += kCT) {
      const int e = i >> 5;
      vl[i] = (uint32_t)c16_s[e & ((1 << VBITS) - 1)] | ((uint32_t)c16_s[e >> VBITS] << 16);
    }
    if (KF == KF_POLAR3 || KF == KF_POLAR4) {
      constexpr int KB = KF == KF_POLAR3 ? 3 : 4;
      uint32_t* kl = reinterpret_cast<uint32_t*>(smem + L::klut);
      constexpr int nk = 1 << (2 * KB);
      constexpr int rep = KF == KF_POLAR4 ? kK4Rep : 32;     // copies of the table (one per lane, or per lane mod rep)
      for (int i = tid; i < nk * rep; i += kCT) {
        const int e = i / rep;
        kl[i] = (uint32_t)c16_s[16 + (e & ((1 << KB) - 1))] | ((uint32_t)c16_s[16 + (e >> KB)] << 16);
      }
    }
  }
  // The query may belong to a kernel that is still running unless the caller vouches
  // for it (q_stable); the shared workspace is first touched after the main loop, and
  // every consumer thread waits for the preceding grid before that.
  if (warp < kConsumerWarps) {
    consumer_barrier();   // tables ready
    if (!a.q_stable) grid_dependency_wait();
  }
  // The query is staged in MMA fragment order when no rotation is needed and its
  // element pairs are naturally aligned; otherwise row by row (rotated in the warp).
  const int q_esize = a.q_dtype == TQ_F32 ? 4 : 2;
  const bool q_direct = ((KF != KF_POLAR3 && KF != KF_POLAR4) || a.q_prerotated) &&
                        reinterpret_cast<uintptr_t>(a.q) % (2 * q_esize) == 0 &&
                        a.q_batch_stride % 2 == 0 && a.q_head_stride % 2 == 0 && a.q_token_stride % 2 == 0;
  if (warp < kConsumerWarps && q_direct) {
    // staged in fragment order [k-step][lane][4 registers]: every element pair is fetched once per
    // CTA, split into f16 high part + residual, and read back with one conflict-free 16-byte load
    uint32_t* qf = reinterpret_cast<uint32_t*>(smem + L::q);
    for (int task = tid; task < 512; task += kConsumerThreads) {
      const int ln = task & 31, up = (task >> 5) & 1, ks = task >> 6;
      const int gg = ln >> 2, tt = ln & 3;
      float2 v = make_float2(0.f, 0.f);
      if (gg < a.rows) {
        const int tok = gg / a.n_rep;
        const int64_t off = b * a.q_batch_stride + (int64_t)(h0 + gg - tok * a.n_rep) * a.q_head_stride +
                            tok * a.q_token_stride + kslot_element<KF>(ks, 2 * tt + 8 * up);
        if (a.q_dtype == TQ_F32) v = *reinterpret_cast<const float2*>(reinterpret_cast<const float*>(a.q) + off);
        else if (a.q_dtype == TQ_F16)
          v = __half22float2(*reinterpret_cast<const __half2*>(reinterpret_cast<const __half*>(a.q) + off));
        else
          v = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(reinterpret_cast<const __nv_bfloat16*>(a.q) + off));
      }
      uint32_t hi, lo;
      split_pair<KF == KF_DENSE_BF16>(v.x, v.y, hi, lo);
      qf[(ks * 32 + ln) * 4 + 2 * up] = hi;
      qf[(ks * 32 + ln) * 4 + 2 * up + 1] = lo;
    }
    consumer_barrier();   // query fragments ready
  }
  // query rows -> shared f16: row r = high part of head r, row 8 + r = residual
  if (warp < kConsumerWarps && !q_direct) {
    __half* qs = reinterpret_cast<__half*>(smem + L::q);
    for (int r = warp; r < 8; r += kConsumerWarps) {
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float x = 0.f;
        if (r < a.rows)
          x = load_any(a.q, a.q_dtype, b * a.q_batch_stride + (int64_t)(h0 + r % a.n_rep) * a.q_head_stride +
                                           (r / a.n_rep) * a.q_token_stride + lane * 4 + j);
        v[j] = x;
      }
      if ((KF == KF_POLAR3 || KF == KF_POLAR4) && !a.q_prerotated) {
#pragma unroll
        for (int j = 0; j < 4; ++j) v[j] *= sign_at(a.k_signs, lane * 4 + j);
        warp_butterfly<4>(v, lane);
      }
      float qsum = 0.f;   // sum of the 16-bit (hi + lo) query values this lane holds
#pragma unroll
      for (int j = 0; j < 4; j += 2) {
        uint32_t hi, lo;
        split_pair<KF == KF_DENSE_BF16>(v[j], v[j + 1], hi, lo);
        *reinterpret_cast<uint32_t*>(qs + r * kDim + lane * 4 + j) = hi;
        *reinterpret_cast<uint32_t*>(qs + (8 + r) * kDim + lane * 4 + j) = lo;
        if (KF == KF_AFFINE8) {
          const float2 hf = __half22float2(*reinterpret_cast<const __half2*>(&hi));
          const float2 lf = __half22float2(*reinterpret_cast<const __half2*>(&lo));
          qsum += (hf.x + lf.x) + (hf.y + lf.y);
        }
      }
      if (KF == KF_AFFINE8) {   // lanes 0-15 hold elements 0-63 (group 0), lanes 16-31 group 1
#pragma unroll
        for (int k = 8; k > 0; k >>= 1) qsum += __shfl_xor_sync(0xffffffffu, qsum, k);
        if ((lane & 15) == 0) qsum_s[r * 2 + (lane >> 4)] = qsum;
      }
    }
    consumer_barrier();   // query rows ready
  }

  const uint8_t* kbase;
  if (is_dense(KF))
    kbase = reinterpret_cast<const uint8_t*>(a.k_data) + (b * a.k_batch_stride + kvh * a.k_head_stride) * 2;
  else if (KF == KF_AFFINE8)
    kbase = reinterpret_cast<const uint8_t*>(a.k_data) + (b * a.k_batch_stride + kvh * a.k_head_stride);
  else
    kbase = reinterpret_cast<const uint8_t*>(a.k_data) + (b * a.k_batch_stride + kvh * a.k_head_stride) * 4;
  // affine keys: per position two fp16 scales and two fp16 biases = one 32-bit word each
  const uint32_t* kscbase = KF == KF_AFFINE8 ? reinterpret_cast<const uint32_t*>(
      reinterpret_cast<const __half*>(a.k_scales) + b * a.ks_batch_stride + kvh * a.ks_head_stride) : nullptr;
  const uint32_t* kbibase = KF == KF_AFFINE8 ? reinterpret_cast<const uint32_t*>(
      reinterpret_cast<const __half*>(a.k_biases) + b * a.ks_batch_stride + kvh * a.ks_head_stride) : nullptr;
  constexpr bool VAFF = VB == 40;
  // packed values: strides in 32-bit words; affine codes: strides in bytes
  const uint8_t* vbase = reinterpret_cast<const uint8_t*>(a.v_data) +
                         (b * a.v_batch_stride + kvh * a.v_head_stride) * (VAFF ? 1 : 4);
  const float* knbase = (is_dense(KF) || KF == KF_AFFINE8)
                            ? nullptr : a.k_norms + b * a.kn_batch_stride + kvh * a.kn_head_stride;
  const float* vnbase = VAFF ? nullptr : a.v_norms + b * a.vn_batch_stride + kvh * a.vn_head_stride;
  // affine values: per position two fp16 scales and two fp16 biases = one 32-bit word each
  const uint32_t* vscbase = VAFF ? reinterpret_cast<const uint32_t*>(
      reinterpret_cast<const __half*>(a.v_scales) + b * a.vs_batch_stride + kvh * a.vs_head_stride) : nullptr;
  const uint32_t* vbibase = VAFF ? reinterpret_cast<const uint32_t*>(
      reinterpret_cast<const __half*>(a.v_biases) + b * a.vs_batch_stride + kvh * a.vs_head_stride) : nullptr;

  // =============================== producer ===============================
  if (warp == kConsumerWarps) {
    // The step's own token (the sequence's last position) is appended by the CTA whose chunk holds
    // it, just before it streams the tile that holds it.
    const bool appends = a.new_v != nullptr && seq - 1 >= pb && seq - 1 < pe && KF != KF_AFFINE8 && !VAFF;
    // K / V may be fetched while preceding kernels are still running only if the caller vouches
    // that they do not write them (kv_stable); likewise the rows to append (q_stable).
    if (!a.kv_stable || (appends && !a.q_stable)) grid_dependency_wait();
    for (int i = 0; i < n_tiles; ++i) {
      const int s = i % kStages;
      const uint32_t ph = (i / kStages) & 1;
      if (i >= kStages && !mbar_wait_relaxed(empty_bar(s), ph ^ 1)) {
        if (lane == 0) atomicExch(tb.status, 1);
        break;
      }
      if (appends && i == n_tiles - 1) {
        const int64_t pn = seq - 1;
        const int64_t koff = b * a.nk_batch_stride + (int64_t)kvh * a.nk_head_stride;
        const int64_t voff = b * a.nv_batch_stride + (int64_t)kvh * a.nv_head_stride;
        if (is_dense(KF)) {          // key row stored as it is (same 16-bit type as the cache)
          if (lane < 16)
            reinterpret_cast<uint4*>(const_cast<uint8_t*>(kbase) + pn * kDenseRowBytes)[lane] =
                reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(a.new_k) + koff * 2)[lane];
        } else if (KF == KF_POLAR3 || KF == KF_POLAR4) {
          constexpr int KB = KF == KF_POLAR3 ? 3 : 4;
          float x[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) x[j] = load_any(a.new_k, a.new_dtype, koff + lane * 4 + j);
          quantize_row_warp<4, KB>(x, a.k_signs, a.k_thr, idx_s,
                                   reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(kbase)) + pn * (KGeom<KF>::row / 4),
                                   const_cast<float*>(knbase) + pn, lane);
        }
        {
          constexpr int VBB = VB == 40 ? 4 : VB;
          float x[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) x[j] = load_any(a.new_v, a.new_dtype, voff + lane * 4 + j);
          quantize_row_warp<4, VBB>(x, a.v_signs, a.v_thr, idx_s,
                                    reinterpret_cast<uint32_t*>(const_cast<uint8_t*>(vbase)) + pn * (VGeom<VB>::row / 4),
                                    const_cast<float*>(vnbase) + pn, lane);
        }
        // the rows were written through the generic proxy; the bulk copies below read them
        // through the async proxy
        __threadfence();
        __syncwarp();
        asm volatile("fence.proxy.async;" ::: "memory");
      }
      const int64_t p0 = pb + (int64_t)i * kTile;
      const int nvp = (int)min((int64_t)kTile, pe - p0);
      const uint32_t st = sbase + L::stage0 + s * L::stage_bytes;
      uint8_t* stg = smem + L::stage0 + s * L::stage_bytes;
      // byte counts moved by bulk copies (multiples of 16); ragged remainders by plain loads
      const uint32_t v_total = nvp * VGeom<VB>::row, v_bulk = v_total & ~15u;
      const uint32_t n_total = nvp * 4, n_bulk = n_total & ~15u;
      const uint32_t k_total = (is_dense(KF) || KF == KF_AFFINE8) ? 0u : (uint32_t)nvp * KGeom<KF>::row;
      const uint32_t k_bulk = k_total & ~15u;
      const uint8_t* vsrc = vbase + p0 * VGeom<VB>::row;
      const uint8_t* ksrc = kbase + p0 * (is_dense(KF) ? 256 : KGeom<KF>::row);
      {
        const int w = lane;   // remainders are at most 3 words each
        if (v_bulk + 4 * w < v_total)
          *reinterpret_cast<uint32_t*>(stg + L::v_off + v_bulk + 4 * w) =
              *reinterpret_cast<const volatile uint32_t*>(vsrc + v_bulk + 4 * w);
        if (n_bulk + 4 * w < n_total) {
          if (VAFF) {
            *reinterpret_cast<uint32_t*>(stg + L::vn_off + n_bulk + 4 * w) = vscbase[p0 + n_bulk / 4 + w];
            *reinterpret_cast<uint32_t*>(stg + L::vn_off + kTile * 4 + n_bulk + 4 * w) = vbibase[p0 + n_bulk / 4 + w];
          } else {
            *reinterpret_cast<float*>(stg + L::vn_off + n_bulk + 4 * w) =
                *reinterpret_cast<const volatile float*>(vnbase + p0 + n_bulk / 4 + w);
          }
        }
        if (KF == KF_POLAR3 || KF == KF_POLAR4) {
          if (k_total != 0 && k_bulk + 4 * w < k_total)
            *reinterpret_cast<uint32_t*>(stg + L::k_off + k_bulk + 4 * w) =
                *reinterpret_cast<const volatile uint32_t*>(ksrc + k_bulk + 4 * w);
          if (n_bulk + 4 * w < n_total)
            *reinterpret_cast<float*>(stg + L::kn_off + n_bulk + 4 * w) =
                *reinterpret_cast<const volatile float*>(knbase + p0 + n_bulk / 4 + w);
        }
        if (KF == KF_AFFINE8) {
          if (n_bulk + 4 * w < n_total) {
            *reinterpret_cast<uint32_t*>(stg + L::kn_off + n_bulk + 4 * w) = kscbase[p0 + n_bulk / 4 + w];
            *reinterpret_cast<uint32_t*>(stg + L::kn_off + kTile * 4 + n_bulk + 4 * w) = kbibase[p0 + n_bulk / 4 + w];
          }
        }
      }
      __syncwarp();
      if (lane == 0) {
        uint32_t tx = v_bulk + (VAFF ? 2 * n_bulk : n_bulk);
        if (is_dense(KF)) tx += (uint32_t)nvp * 256u;
        else if (KF == KF_AFFINE8) tx += (uint32_t)nvp * 128u + 2 * n_bulk;
        else tx += k_bulk + n_bulk;
        mbar_arrive_expect_tx(full_bar(s), tx);
        if (is_dense(KF)) bulk_g2s(st + L::k_off, ksrc, (uint32_t)nvp * 256u, full_bar(s));
        if (KF == KF_AFFINE8) {
          bulk_g2s(st + L::k_off, ksrc, (uint32_t)nvp * 128u, full_bar(s));
          if (n_bulk) bulk_g2s(st + L::kn_off, kscbase + p0, n_bulk, full_bar(s));
          if (n_bulk) bulk_g2s(st + L::kn_off + kTile * 4, kbibase + p0, n_bulk, full_bar(s));
        }
        if (v_bulk) bulk_g2s(st + L::v_off, vsrc, v_bulk, full_bar(s));
        if (VAFF) {
          if (n_bulk) bulk_g2s(st + L::vn_off, vscbase + p0, n_bulk, full_bar(s));
          if (n_bulk) bulk_g2s(st + L::vn_off + kTile * 4, vbibase + p0, n_bulk, full_bar(s));
        } else if (n_bulk) {
          bulk_g2s(st + L::vn_off, vnbase + p0, n_bulk, full_bar(s));
        }
        if (KF == KF_POLAR3 || KF == KF_POLAR4) {
          if (k_bulk) bulk_g2s(st + L::k_off, ksrc, k_bulk, full_bar(s));
          if (n_bulk) bulk_g2s(st + L::kn_off, knbase + p0, n_bulk, full_bar(s));
        }
      }
      __syncwarp();
    }
    return;
  }

  // =============================== consumers ===============================
  // query fragments in the k-slot order of this key format
  uint32_t aq[8][4];
  float qsum0 = 0.f, qsum1 = 0.f;   // affine keys: sums of head g's query over elements 0-63 / 64-127
  if (q_direct) {
    const uint4* qf = reinterpret_cast<const uint4*>(smem + L::q);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const uint4 f = qf[ks * 32 + lane];
      aq[ks][0] = f.x; aq[ks][1] = f.y; aq[ks][2] = f.z; aq[ks][3] = f.w;
      if (KF == KF_AFFINE8) {
        const float2 a0 = __half22float2(*reinterpret_cast<const __half2*>(&f.x));
        const float2 a1 = __half22float2(*reinterpret_cast<const __half2*>(&f.y));
        const float2 a2 = __half22float2(*reinterpret_cast<const __half2*>(&f.z));
        const float2 a3 = __half22float2(*reinterpret_cast<const __half2*>(&f.w));
        const float sum = ((a0.x + a1.x) + (a0.y + a1.y)) + ((a2.x + a3.x) + (a2.y + a3.y));
        if (ks < 4) qsum0 += sum; else qsum1 += sum;
      }
    }
    if (KF == KF_AFFINE8) {
      qsum0 += __shfl_xor_sync(0xffffffffu, qsum0, 1);
      qsum0 += __shfl_xor_sync(0xffffffffu, qsum0, 2);
      qsum1 += __shfl_xor_sync(0xffffffffu, qsum1, 1);
      qsum1 += __shfl_xor_sync(0xffffffffu, qsum1, 2);
    }
  } else {
    const __half* qs = reinterpret_cast<const __half*>(smem + L::q);
#pragma unroll
    for (int ks = 0; ks < 8; ++ks) {
      const int e_lo = kslot_element<KF>(ks, 2 * t);
      const int e_hi = kslot_element<KF>(ks, 2 * t + 8);
      aq[ks][0] = *reinterpret_cast<const uint32_t*>(qs + g * kDim + e_lo);
      aq[ks][1] = *reinterpret_cast<const uint32_t*>(qs + (g + 8) * kDim + e_lo);
      aq[ks][2] = *reinterpret_cast<const uint32_t*>(qs + g * kDim + e_hi);
      aq[ks][3] = *reinterpret_cast<const uint32_t*>(qs + (g + 8) * kDim + e_hi);
    }
    if (KF == KF_AFFINE8) {
      qsum0 = qsum_s[2 * g];
      qsum1 = qsum_s[2 * g + 1];
    }
  }
  // V side: this thread's 16 elements are 16g .. 16g+15 (8 pairs)
  const uint32_t lane4 = lane * 4;
  const int v_w0 = (16 * g) / 10;                       // first word holding element 16g (3-bit rows)
  const int v_s0 = 3 * ((16 * g) % 10);                 // its bit offset inside that word
  const int v_w2 = min(v_w0 + 2, 12);

  float o[8][4];
#pragma unroll
  for (int j = 0; j < 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  int active_count = 0;             // positions whose values this warp accumulated (reported when asked for)
  // value skipping across splits: the hint words are shared by the CTAs of the group and put back to zero by the
  // CTA that merges it, so they may only be used by a call that is alone on its workspace while it runs (its own
  // workspace, or a call that has already waited for its predecessor)
  const bool use_group_hint = !PLAIN && a.sparse_thr > 0.f && tb.hints != nullptr && (a.ws_exclusive || !a.q_stable);
  uint32_t* group_hint = tb.hints + 8 * (b * a.n_kv_heads + kvh);
  float bias_run[2] = {0.f, 0.f};   // affine values: sum of weight x bias per element group (head g, this lane's positions)
  const int pw = 16 * warp;   // first position of this warp inside a tile

  const int span = (int)(pe - pb);          // positions of this chunk (at most one chunk: fits 32 bits)
  for (int i = 0; i < n_tiles; ++i) {
    const int s = i % kStages;
    if (!mbar_wait(full_bar(s), (i / kStages) & 1)) {
      // Bounded wait gave up: flag it for the whole CTA.  Every warp still walks through the
      // epilogue's barriers and the split counter, so nobody is left waiting and the counters
      // return to zero; the result is invalid and the status word says so.
      if (lane == 0) {
        atomicExch(tb.status, 2);
        abort_s = 1;
      }
      break;
    }
    const uint32_t st = sbase + L::stage0 + s * L::stage_bytes;
    const int nvp = min(kTile, span - i * kTile);
    // several query tokens: token t (row g's) does not see the sequence's last q_tokens - 1 - t positions
    // (recomputed per tile so that the one-token path carries nothing extra through the loop)
    int nvp_row = nvp;
    if (!PLAIN && a.q_tokens > 1 && g < a.rows) {
      const int64_t sq = a.seq_lens != nullptr ? max((int64_t)0, min((int64_t)a.seq_lens[blockIdx.z], a.seq_len)) : a.seq_len;
      const int64_t tile0 = (int64_t)blockIdx.x * a.chunk + (int64_t)i * kTile;
      nvp_row = min(nvp, (int)min((int64_t)(2 * kTile), sq - tile0) - (a.q_tokens - 1 - g / a.n_rep));
    }

    // value skipping: what the other CTAs of the group have seen so far, fetched now so that the latency is
    // gone by the time the tile's own scores exist (only real scores are ever written there, so whatever a
    // relaxed read returns is a valid lower bound of the head's largest score)
    uint32_t group_key = 0u;
    if (use_group_hint) asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(group_key) : "l"(group_hint + g));

    // ---------------- scores ----------------
    float sc[2][4];
#pragma unroll
    for (int ng = 0; ng < 2; ++ng) {
      sc[ng][0] = sc[ng][1] = sc[ng][2] = sc[ng][3] = 0.f;
      const int prow = pw + 8 * ng + g;
      if (is_dense(KF)) {
        const uint32_t row = st + L::k_off + prow * kDenseRowBytes + t * 16;
        float sc2[4] = {0.f, 0.f, 0.f, 0.f};   // second accumulator: two independent MMA chains
        uint4 r[4];
#pragma unroll
        for (int it = 0; it < 4; ++it) r[it] = lds128(row + it * 64);
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          if (KF == KF_DENSE_BF16) {
            mma16816_bf16(sc[ng], aq[2 * it], r[it].x, r[it].y);
            mma16816_bf16(sc2, aq[2 * it + 1], r[it].z, r[it].w);
          } else {
            mma16816(sc[ng], aq[2 * it], r[it].x, r[it].y);
            mma16816(sc2, aq[2 * it + 1], r[it].z, r[it].w);
          }
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) sc[ng][c] += sc2[c];
      } else if (KF == KF_AFFINE8) {
        // codes -> f16 (1024 + code) with one PRMT per pair; one accumulator per 64-element group;
        // the offset and the per-position scale / bias are applied after the MMA
        const uint32_t row = st + L::k_off + prow * 128 + t * 16;
        float g1[4] = {0.f, 0.f, 0.f, 0.f};
        const uint4 r0 = lds128(row), r1 = lds128(row + 64);
        const uint32_t w0[4] = {r0.x, r0.y, r0.z, r0.w}, w1[4] = {r1.x, r1.y, r1.z, r1.w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          mma16816(sc[ng], aq[w], __byte_perm(w0[w], 0x64646464u, 0x4140), __byte_perm(w0[w], 0x64646464u, 0x4342));
          mma16816(g1, aq[4 + w], __byte_perm(w1[w], 0x64646464u, 0x4140), __byte_perm(w1[w], 0x64646464u, 0x4342));
        }
        const float q0 = qsum0, q1 = qsum1;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int pos = pw + 8 * ng + 2 * t + c;
          const __half2 sc2h = *reinterpret_cast<const __half2*>(smem + L::stage0 + s * L::stage_bytes + L::kn_off + pos * 4);
          const __half2 bi2h = *reinterpret_cast<const __half2*>(smem + L::stage0 + s * L::stage_bytes + L::kn_off + kTile * 4 + pos * 4);
          const float d0 = (sc[ng][c] + sc[ng][c + 2]) - 1024.f * q0;     // sum_e q_e * code_e, group 0
          const float d1 = (g1[c] + g1[c + 2]) - 1024.f * q1;
          const float dot = __low2float(sc2h) * d0 + __low2float(bi2h) * q0 +
                            __high2float(sc2h) * d1 + __high2float(bi2h) * q1;
          sc[ng][c] = dot;          // the generic post-processing below adds [c] and [c + 2]
          sc[ng][c + 2] = 0.f;
        }
      } else if (KF == KF_POLAR4) {
        const uint4 w4 = lds128(st + L::k_off + prow * 64 + t * 16);
        const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
        float sc2[4] = {0.f, 0.f, 0.f, 0.f};   // second accumulator: two independent MMA chains
#pragma unroll
        for (int wi = 0; wi < 4; ++wi) {
          // byte address of pair entry e in this lane's copy: e * (kK4Rep * 4) + (lane mod kK4Rep) * 4
          constexpr int esh = kK4Rep == 32 ? 7 : 6;
          constexpr uint32_t emask = 0xFFu << esh;
          const uint32_t lk = (lane & (kK4Rep - 1)) * 4;
          const uint32_t a0 = ((w[wi] << esh) & emask) | lk;
          const uint32_t a1 = ((w[wi] >> (8 - esh)) & emask) | lk;
          const uint32_t a2 = ((w[wi] >> (16 - esh)) & emask) | lk;
          const uint32_t a3 = ((w[wi] >> (24 - esh)) & emask) | lk;
          mma16816(sc[ng], aq[2 * wi], lut_ld(smem + L::klut, a0), lut_ld(smem + L::klut, a1));
          mma16816(sc2, aq[2 * wi + 1], lut_ld(smem + L::klut, a2), lut_ld(smem + L::klut, a3));
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) sc[ng][c] += sc2[c];
      } else {
        const uint32_t row = st + L::k_off + prow * 52;
        uint32_t w[3];
        w[0] = lds32(row + 12 * t);
        w[1] = lds32(row + 12 * t + 4);
        w[2] = lds32(row + 12 * t + 8);
        const uint32_t w12 = lds32(row + 48) >> (6 * t);
        uint32_t bq[16];
#pragma unroll
        for (int pi = 0; pi < 15; ++pi) {
          const uint32_t ww = w[pi / 5];
          const int sh = 6 * (pi % 5) - 7;
          bq[pi] = ((sh >= 0 ? (ww >> sh) : (ww << (-sh))) & 0x1F80u) | lane4;
        }
        bq[15] = ((w12 << 7) & 0x1F80u) | lane4;
        float sc2[4] = {0.f, 0.f, 0.f, 0.f};   // second accumulator: two independent MMA chains
#pragma unroll
        for (int ks = 0; ks < 8; ks += 2) {
          mma16816(sc[ng], aq[ks], lut_ld(smem + L::klut, bq[2 * ks]), lut_ld(smem + L::klut, bq[2 * ks + 1]));
          mma16816(sc2, aq[ks + 1], lut_ld(smem + L::klut, bq[2 * ks + 2]), lut_ld(smem + L::klut, bq[2 * ks + 3]));
        }
#pragma unroll
        for (int c = 0; c < 4; ++c) sc[ng][c] += sc2[c];
      }
    }

    // ---------------- softmax (log2 domain) ----------------
    // this thread: head g, positions pw + 8*ng + 2t + c
    // s2v: score + log2 of the value row's norm (packed values), so that the f16 weights stay <= 2^8
    // for any norm; affine values carry their scale on the other operand and use the plain score
    float s2[2][2], s2v[2][2], vbias[2][2][2];
    uint32_t vscw[2][2];                       // affine values: (scale group 0, scale group 1) of the position
    float m_tile = -INFINITY;
#pragma unroll
    for (int ng = 0; ng < 2; ++ng)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const int pos = pw + 8 * ng + 2 * t + c;
        float v = (sc[ng][c] + sc[ng][c + 2]) * tb.k_post;
        if (KF == KF_POLAR3 || KF == KF_POLAR4) v *= lds_f32(st + L::kn_off + pos * 4);
        const bool valid = pos < nvp_row;
        s2[ng][c] = valid ? v : -INFINITY;
        if (VAFF) {
          vscw[ng][c] = valid ? lds32(st + L::vn_off + pos * 4) : 0u;   // stale words past the end must not reach the MMA
          const uint32_t bw = lds32(st + L::vn_off + kTile * 4 + pos * 4);
          const __half2 vbi = *reinterpret_cast<const __half2*>(&bw);
          vbias[ng][c][0] = valid ? __low2float(vbi) : 0.f;
          vbias[ng][c][1] = valid ? __high2float(vbi) : 0.f;
          s2v[ng][c] = s2[ng][c];
        } else {
          const float vn = lds_f32(st + L::vn_off + pos * 4);
          s2v[ng][c] = valid ? v + lg2(fmaxf(vn, 1e-26f)) : -INFINITY;
        }
        m_tile = fmaxf(m_tile, s2v[ng][c]);
      }
    m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 1));
    m_tile = fmaxf(m_tile, __shfl_xor_sync(0xffffffffu, m_tile, 2));
    const bool need = m_tile > m_run + kRescaleThreshold;   // also true for the first finite tile
    if (__any_sync(0xffffffffu, need)) {
      const float alpha = need ? (m_run == -INFINITY ? 0.f : ex2(m_run - m_tile)) : 1.f;
      if (need) m_run = m_tile;
      l_run *= alpha;
      if (VAFF) {
        bias_run[0] *= alpha;
        bias_run[1] *= alpha;
      }
      const float al0 = __shfl_sync(0xffffffffu, alpha, 8 * t);        // head 2t lives in lanes 8t..8t+3
      const float al1 = __shfl_sync(0xffffffffu, alpha, 8 * t + 4);    // head 2t + 1
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        o[j][0] *= al0; o[j][1] *= al1; o[j][2] *= al0; o[j][3] *= al1;
      }
    }
    const float m_use = m_run == -INFINITY ? 0.f : m_run;
    float pv[2][2];
#pragma unroll
    for (int ng = 0; ng < 2; ++ng)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        pv[ng][c] = ex2(s2v[ng][c] - m_use);
        if (VAFF) {
          l_run += pv[ng][c];
          bias_run[0] += pv[ng][c] * vbias[ng][c][0];     // the bias of a group reaches all of its elements alike
          bias_run[1] += pv[ng][c] * vbias[ng][c][1];
        } else {
          l_run += ex2(s2[ng][c] - m_use);
        }
      }
    // Value skipping: the final softmax weight of a position is at most exp(score - running max) /
    // running sum (both only grow), so a tile whose every weight is below the threshold by that bound,
    // for every head of the group, contributes nothing the reference would keep.
    bool skip_values = false;
    if (!PLAIN && a.sparse_thr > 0.f) {
      float smax = -INFINITY;                            // largest score among this thread's positions
#pragma unroll
      for (int ng = 0; ng < 2; ++ng)
#pragma unroll
        for (int c = 0; c < 2; ++c) smax = fmaxf(smax, s2[ng][c]);
      float lq = l_run;                                  // running sum of head g in this warp: the quad's lanes
      lq += __shfl_xor_sync(0xffffffffu, lq, 1);
      lq += __shfl_xor_sync(0xffffffffu, lq, 2);
      // the log-sum-exp of a head is at least any single score: the largest one seen by any warp of
      // the CTA so far is a second lower bound (shared through hint_s)
      float sq = fmaxf(smax, __shfl_xor_sync(0xffffffffu, smax, 1));
      sq = fmaxf(sq, __shfl_xor_sync(0xffffffffu, sq, 2));
      float hint = from_ordered_int(*reinterpret_cast<volatile int*>(&hint_s[g]));
      if (group_key != 0u) hint = fmaxf(hint, from_ordered_int((int)(group_key ^ 0x80000000u)));
      if (t == 0 && g < a.rows && sq > hint) {           // rare once the large scores are in
        atomicMax(&hint_s[g], ordered_int(sq));
        if (use_group_hint) atomicMax(group_hint + g, (uint32_t)ordered_int(sq) ^ 0x80000000u);
      }
      hint = fmaxf(hint, sq);
      const bool below = smax == -INFINITY || ex2(smax - m_use) < a.sparse_thr * lq || ex2(smax - hint) < a.sparse_thr;
      skip_values = __all_sync(0xffffffffu, g >= a.rows || below);
    }
    if (!PLAIN && !skip_values && pw < nvp) active_count += min(16, nvp - pw);   // one atomic per warp, after the loop
    if (!skip_values) {
    const uint32_t pb0 = pack_h2(pv[0][0], pv[0][1]);   // k = 2t, 2t+1      (positions pw + 2t ..)
    const uint32_t pb1 = pack_h2(pv[1][0], pv[1][1]);   // k = 2t+8, 2t+9    (positions pw + 8 + 2t ..)
    // affine values: this lane's 16 elements lie in group g / 4; its scales for the two position pairs
    const uint32_t grp_sel = (g >> 2) ? 0x7632u : 0x5410u;
    const uint32_t vs0 = VAFF ? __byte_perm(vscw[0][0], vscw[0][1], grp_sel) : 0u;
    const uint32_t vs1 = VAFF ? __byte_perm(vscw[1][0], vscw[1][1], grp_sel) : 0u;

    // ---------------- values ----------------
    // positions handled by this thread as MMA k: pw + 2t, +1 and pw + 8 + 2t, +1
    uint32_t xlo[4], xhi[4];
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const int pos = pw + 2 * t + (q4 & 1) + 8 * (q4 >> 1);
      if (VB == 3) {
        const uint32_t row = st + L::v_off + pos * 52;
        const uint32_t w0 = lds32(row + 4 * v_w0), w1 = lds32(row + 4 * v_w0 + 4), w2 = lds32(row + 4 * v_w2);
        // 48-bit stream of this thread's 16 codes, element 16g first
        xlo[q4] = (w0 >> v_s0) | (w1 << (30 - v_s0));
        xhi[q4] = (w1 >> (2 + v_s0)) | (w2 << (28 - v_s0));
      } else {
        const uint2 w = lds64(st + L::v_off + pos * 64 + 8 * g);
        xlo[q4] = w.x;
        xhi[q4] = w.y;
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      uint32_t lv[4];
#pragma unroll
      for (int q4 = 0; q4 < 4; ++q4) {
        uint32_t addr;
        if (VB == 3) {
          // pair j = bits [6j, 6j+6) of the stream; LUT byte address = idx * 128 + lane * 4
          if (j == 0) addr = (xlo[q4] << 7) & 0x1F80u;
          else if (j == 1) addr = (xlo[q4] << 1) & 0x1F80u;
          else if (j < 5) addr = (xlo[q4] >> (6 * j - 7)) & 0x1F80u;
          else if (j == 5) addr = (__funnelshift_r(xlo[q4], xhi[q4], 23)) & 0x1F80u;
          else if (j == 6) addr = (xhi[q4] << 3) & 0x1F80u;     // stream bits 36..41 = xhi bits 4..9
          else addr = (xhi[q4] >> 3) & 0x1F80u;                  // stream bits 42..47 = xhi bits 10..15
        } else {
          const uint32_t w = j < 4 ? xlo[q4] : xhi[q4];
          const int sh = 8 * (j & 3) - 7;
          addr = (sh >= 0 ? (w >> sh) : (w << 7)) & 0x7F80u;
        }
        lv[q4] = lut_ld(smem + L::vlut, addr | lane4);
      }
      uint32_t af[4];
      af[0] = __byte_perm(lv[0], lv[1], 0x5410);   // element 16g+2j,   positions 2t, 2t+1
      af[1] = __byte_perm(lv[0], lv[1], 0x7632);   // element 16g+2j+1, positions 2t, 2t+1
      af[2] = __byte_perm(lv[2], lv[3], 0x5410);   // element 16g+2j,   positions 2t+8, 2t+9
      af[3] = __byte_perm(lv[2], lv[3], 0x7632);
      if (VAFF) {   // code (exact in f16) x scale of (position, group)
        af[0] = hmul2_bits(af[0], vs0);
        af[1] = hmul2_bits(af[1], vs0);
        af[2] = hmul2_bits(af[2], vs1);
        af[3] = hmul2_bits(af[3], vs1);
      }
      mma16816(o[j], af, pb0, pb1);
    }
    }   // !skip_values
    __syncwarp();
    if (lane == 0) mbar_arrive(empty_bar(s));
  }

  if (!PLAIN && a.active_positions != nullptr && lane == 0 && active_count > 0)
    atomicAdd(a.active_positions + b * a.n_kv_heads + kvh, active_count);

  // ---------------- CTA epilogue: one exchange through shared memory ----------------
  // Every warp writes its (o[32], m, l) once, [warp][value][lane] (conflict free);
  // after one barrier each thread sums a fixed slice of the 32 accumulator values
  // over the source warps and stores its share of the split's partial state.
  consumer_barrier();   // every consumer is done with the ring
  float* xch = reinterpret_cast<float*>(smem + L::stage0);               // [warp][xch_rows][32]
  {
    constexpr int R = L::xch_rows;
    float* dst = xch + warp * R * 32 + lane;
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int c = 0; c < 4; ++c) dst[(j * 4 + c) * 32] = o[j][c];
    dst[32 * 32] = m_run;
    dst[33 * 32] = l_run;
    if (VAFF) {   // bias sums of head g, both element groups, summed over the four lanes of the head
#pragma unroll
      for (int gi = 0; gi < 2; ++gi) {
        float bsum = bias_run[gi];
        bsum += __shfl_xor_sync(0xffffffffu, bsum, 1);
        bsum += __shfl_xor_sync(0xffffffffu, bsum, 2);
        dst[(34 + gi) * 32] = bsum;
      }
    }
  }
  consumer_barrier();
  // A workspace shared with the preceding launch (partial states, counters) is written from here
  // on, so every consumer thread first waits for that launch to complete.  A call with a workspace of
  // its own (ws_exclusive) and stable inputs depends on nothing: it does not wait here, and the tails
  // of consecutive launches (hand-over, merge) overlap like their main loops do.
  const bool independent = a.kv_stable && a.q_stable && a.ws_exclusive;
  if (a.q_stable && !independent) grid_dependency_wait();
  const int64_t n_rows = (int64_t)a.batch * a.n_kv_heads * a.rows;
  const int64_t row0 = ((int64_t)b * a.n_kv_heads + kvh) * a.rows;
  {
    constexpr int R = L::xch_rows;
    // rescale factors of the source warps for this thread's two heads (2t, 2t+1)
    float f0[kConsumerWarps], f1[kConsumerWarps];
    float m0 = -INFINITY, m1 = -INFINITY;
#pragma unroll
    for (int sw = 0; sw < kConsumerWarps; ++sw) {
      f0[sw] = xch[(sw * R + 32) * 32 + 8 * t];        // m of head 2t   (any lane with g == 2t)
      f1[sw] = xch[(sw * R + 32) * 32 + 8 * t + 4];    // m of head 2t+1
      m0 = fmaxf(m0, f0[sw]);
      m1 = fmaxf(m1, f1[sw]);
    }
#pragma unroll
    for (int sw = 0; sw < kConsumerWarps; ++sw) {
      f0[sw] = f0[sw] == -INFINITY ? 0.f : ex2(f0[sw] - m0);
      f1[sw] = f1[sw] == -INFINITY ? 0.f : ex2(f1[sw] - m1);
    }
    // affine values: weighted bias of this lane's element group (g / 4) for its two heads
    float bias0 = 0.f, bias1 = 0.f;
    if (VAFF) {
#pragma unroll
      for (int sw = 0; sw < kConsumerWarps; ++sw) {
        bias0 += xch[(sw * R + 34 + (g >> 2)) * 32 + 8 * t] * f0[sw];
        bias1 += xch[(sw * R + 34 + (g >> 2)) * 32 + 8 * t + 4] * f1[sw];
      }
    }
    float* acc0 = a.part_acc + ((int64_t)split * n_rows + row0) * kDim;
#pragma unroll
    for (int kk = 0; kk < (32 + kConsumerWarps - 1) / kConsumerWarps; ++kk) {
      const int k = warp + kConsumerWarps * kk;          // accumulator value index j * 4 + c
      if (k < 32) {
        const int j = k >> 2, c = k & 3;
        float v = 0.f;
#pragma unroll
        for (int sw = 0; sw < kConsumerWarps; ++sw)
          v += xch[(sw * R + k) * 32 + lane] * ((c & 1) ? f1[sw] : f0[sw]);
        const int head = 2 * t + (c & 1);
        if (head < a.rows)
          acc0[head * kDim + 16 * g + 2 * j + (c >> 1)] = v * tb.v_post + (VAFF ? ((c & 1) ? bias1 : bias0) : 0.f);
      }
    }
    if (warp == kConsumerWarps - 1) {
      // l and m of head g: this lane's own head needs its own factors
      float mg = -INFINITY;
#pragma unroll
      for (int sw = 0; sw < kConsumerWarps; ++sw) mg = fmaxf(mg, xch[(sw * R + 32) * 32 + lane]);
      float lg = 0.f;
#pragma unroll
      for (int sw = 0; sw < kConsumerWarps; ++sw) {
        const float ms = xch[(sw * R + 32) * 32 + lane];
        lg += xch[(sw * R + 33) * 32 + lane] * (ms == -INFINITY ? 0.f : ex2(ms - mg));
      }
      lg += __shfl_xor_sync(0xffffffffu, lg, 1);
      lg += __shfl_xor_sync(0xffffffffu, lg, 2);
      if (t == 0 && g < a.rows) {
        a.part_m[(int64_t)split * n_rows + row0 + g] = mg == -INFINITY ? -INFINITY : mg * 0.6931471805599453f;
        a.part_l[(int64_t)split * n_rows + row0 + g] = lg;
      }
    }
  }
  // ---------------- merge across splits, no waiting anywhere ----------------
  // Every CTA publishes its partial and bumps the group's counter with one release /
  // acquire atomic (the barrier in front makes the whole CTA's stores precede it); the CTA
  // that completes the count owns the merge and resets the counter, so counters are zero
  // between calls.
  const int count = tb.splits;
  consumer_barrier();
  if (tid == 0) {
    int elected = 1;
    if (count > 1) {
      int* ctr = tb.counters + (b * a.n_kv_heads + kvh);
      int prev;
      asm volatile("atom.acq_rel.gpu.global.add.s32 %0, [%1], 1;" : "=r"(prev) : "l"(ctr) : "memory");
      elected = prev == count - 1;
      if (elected) *ctr = 0;
    }
    elected_s = elected;
  }
  consumer_barrier();
  if (!elected_s) return;
  if (use_group_hint && tid < 8) group_hint[tid] = 0u;   // every CTA of the group is past its loop: zero between calls
  // A push into peer slots that an exchange still in flight may be reading (a small ring of slots) has to
  // come after the launch in front of this one - the gated merge that reads them - has completed.
  if (independent && tb.n_peers > 0 && !tb.peer_unordered) grid_dependency_wait();

  // The merge reads every part's state straight from L2 into registers.  Shared scratch
  // (the ring is free): weights [8][kMaxParts], m* [8], l* [8].
  float* wgt = reinterpret_cast<float*>(smem + L::stage0);
  float* mst = wgt + 8 * kMaxParts;
  float* lst = mst + 8;
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  // parts: m / l at pm / pl + i * ml_stride + row, acc rows at pacc + i * acc_stride + row * 128
  auto merge_pass = [&](const float* pm, const float* pl, const float* pacc, int64_t ml_stride, int64_t acc_stride,
                        int cnt, bool final_out, bool poisoned) {
    for (int r = warp; r < a.rows; r += kConsumerWarps) {
      // lane i (+32, +64) holds part i: m* = max over parts with l > 0, weight = e^(m - m*)
      float mi[3], li[3];
#pragma unroll
      for (int s3 = 0; s3 < 3; ++s3) {
        const int i = lane + 32 * s3;
        const bool on = i < cnt;
        li[s3] = on ? __ldcg(pl + (int64_t)i * ml_stride + row0 + r) : 0.f;
        mi[s3] = on ? __ldcg(pm + (int64_t)i * ml_stride + row0 + r) : -INFINITY;
      }
      float mx = -INFINITY;
#pragma unroll
      for (int s3 = 0; s3 < 3; ++s3)
        if (li[s3] > 0.f) mx = fmaxf(mx, mi[s3]);
      mx = warp_max(mx);
      float lsum = 0.f;
#pragma unroll
      for (int s3 = 0; s3 < 3; ++s3) {
        const int i = lane + 32 * s3;
        const float w = li[s3] > 0.f ? __expf(mi[s3] - mx) : 0.f;
        if (i < cnt) wgt[r * kMaxParts + i] = w;
        lsum += li[s3] * w;
      }
      lsum = warp_sum(lsum);
      if (lane == 0) {
        mst[r] = mx;
        lst[r] = poisoned ? __int_as_float(0x7fc00000) : lsum;   // a rank never pushed: hand out NaN, not a partial merge
      }
    }
    consumer_barrier();
    const int64_t pstride = acc_stride / 4;               // float4s between consecutive parts
    // warp w owns rows w, w + kConsumerWarps, ...; a lane owns elements 4*lane .. 4*lane+3 of its row
    for (int r = warp; r < a.rows; r += kConsumerWarps) {
      float4 acc4 = zero4;
      const float4* src = reinterpret_cast<const float4*>(pacc + (row0 + r) * kDim) + lane;
      const float* wr = wgt + r * kMaxParts;
      for (int i0 = 0; i0 < cnt; i0 += kMergeBatch) {
        float4 v[kMergeBatch];
#pragma unroll
        for (int j = 0; j < kMergeBatch; ++j)
          v[j] = i0 + j < cnt ? __ldcg(src + (int64_t)(i0 + j) * pstride) : zero4;
#pragma unroll
        for (int j = 0; j < kMergeBatch; ++j) {
          const float wi = i0 + j < cnt ? wr[i0 + j] : 0.f;
          acc4.x += v[j].x * wi; acc4.y += v[j].y * wi; acc4.z += v[j].z * wi; acc4.w += v[j].w * wi;
        }
      }
      write_row<VAFF>(a, tb, b, h0, r, row0 + r, acc4, mst[r], lst[r], lane, final_out);
    }
  };
  merge_pass(a.part_m, a.part_l, a.part_acc, n_rows, n_rows * kDim, count, tb.out_mode == 0, false);
  if (tb.out_mode != 0 && tb.n_peers > 0) {
    // every row of this (batch, kv head) group is on its way: one thread fences at system scope (the
    // barrier makes the other threads' stores precede it) and tells each peer
    consumer_barrier();
    if (tid == 0) {
      __threadfence_system();
#pragma unroll
      for (int p = 0; p < 8; ++p)
        if (p < tb.n_peers) atomicAdd_system(tb.peer_counter[p], 1u);
    }
  }
  if (tb.out_mode == 2) {
    // The ranks' rows of this exchange arrive in this GPU's own slot; thread e waits for rank e's counter
    // (bounded by a time limit on the GPU-wide timer and by an iteration count).
    __shared__ int gather_failed_s;
    if (tid == 0) gather_failed_s = 0;
    consumer_barrier();
    if (tid < tb.g_ranks) {
      bool seen = false;
      unsigned long long t0;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
      for (uint32_t it = 0; it < (1u << 28) && !seen; ++it) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(tb.g_flags + tid) : "memory");
        seen = v >= (uint32_t)tb.g_expect;
        if (!seen) {
          __nanosleep(40);
          unsigned long long t1;
          asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
          if (t1 - t0 > tb.g_limit_ns) break;
        }
      }
      if (!seen) {
        atomicExch(tb.status, 21 + tid);
        gather_failed_s = 1;
      }
    }
    consumer_barrier();
    // the CTA of this rank that is last past the wait puts the counters back to zero for the next use
    if (tid == 0) {
      const uint32_t prev = atomicAdd(tb.g_flags + tb.g_ranks, 1u);
      if (prev == (uint32_t)tb.g_expect - 1) {
        for (int i = 0; i <= tb.g_ranks; ++i)
          asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(tb.g_flags + i), "r"(0u) : "memory");
      }
    }
    merge_pass(tb.g_m, tb.g_l, tb.g_acc, tb.g_stride, tb.g_stride, tb.g_ranks, true, gather_failed_s != 0);
  }
  // An independent launch still must not complete before its predecessor has: later work on the
  // stream is ordered after this grid only.  The CTA that merged is the last to leave; it waits.
  if (independent && tid == 0) grid_dependency_wait();
}

// ---- host side: scaled f16 codebooks --------------------------------------------------
struct ScaledBook {
  float key[16];
  int n;
  uint16_t c16[16];
  float beta;
};

// f16 has an 11-bit significand; rounding the centroids directly would leave a
// fixed relative error of up to 2^-12 on each.  A common factor beta in [1, 2)
// is searched so that every beta * c_i lands (almost) on an f16 value; 1/beta is
// applied in float32 after the MMA.
static void scale_codebook(const float* c, int n, ScaledBook* out) {
  static std::mutex mu;
  static ScaledBook cache[8];
  static int n_cached = 0;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < n_cached; ++i) {
    if (cache[i].n == n && memcmp(cache[i].key, c, n * sizeof(float)) == 0) {
      *out = cache[i];
      return;
    }
  }
  float best_beta = 1.f;
  double best_err = 1e30;
  for (int step = 0; step < (1 << 16); ++step) {
    const float beta = 1.0f + step * (1.0f / 65536.0f);
    double worst = 0.0;
    for (int i = 0; i < n && worst < best_err; ++i) {
      if (c[i] == 0.f) continue;
      const double exact = (double)beta * (double)c[i];
      const double got = (double)__half2float(__float2half_rn((float)exact));
      const double rel = fabs(got - exact) / fabs(exact);
      if (rel > worst) worst = rel;
    }
    if (worst < best_err) {
      best_err = worst;
      best_beta = beta;
    }
  }
  ScaledBook sb;
  memset(&sb, 0, sizeof(sb));
  sb.n = n;
  memcpy(sb.key, c, n * sizeof(float));
  sb.beta = best_beta;
  for (int i = 0; i < n; ++i) {
    const __half h = __float2half_rn(best_beta * c[i]);
    sb.c16[i] = *reinterpret_cast<const uint16_t*>(&h);
  }
  if (n_cached < 8) cache[n_cached++] = sb;
  *out = sb;
}

static int g_ctas_per_sm_seen = -1;   // occupancy the runtime reports for the variant set up last


template <int KF, int VB, bool PLAIN>
static int launch_variant_p(const FlashArgs& a, const MmaTables& tb, int splits, cudaStream_t st) {
  using L = Layout<KF, VB>;
  static bool attr_done[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !attr_done[dev]) {
    cudaError_t e = cudaFuncSetAttribute(flash_mma_kernel<KF, VB, PLAIN>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, L::total);
    if (e == cudaSuccess)   // two CTAs per SM need the full shared-memory carve-out
      e = cudaFuncSetAttribute(flash_mma_kernel<KF, VB, PLAIN>, cudaFuncAttributePreferredSharedMemoryCarveout,
                               cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return set_error(TQ_ERR_LAUNCH, "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_done[dev] = true;
    int n = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, flash_mma_kernel<KF, VB, PLAIN>, kThreads, L::total) == cudaSuccess)
      g_ctas_per_sm_seen = n;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(splits, a.n_kv_heads, a.batch);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = L::total;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;   // may start while its predecessor drains
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, flash_mma_kernel<KF, VB, PLAIN>, a, tb);
  if (e != cudaSuccess) return set_error(TQ_ERR_LAUNCH, "tq_flash_decode (mma): %s", cudaGetErrorString(e));
  return check_launch("tq_flash_decode (mma)");
}

template <int KF, int VB>
static int launch_variant(const FlashArgs& a, const MmaTables& tb, int splits, cudaStream_t st) {
  const bool plain = !(a.sparse_thr > 0.f) && a.active_positions == nullptr && a.q_tokens <= 1;
  return plain ? launch_variant_p<KF, VB, true>(a, tb, splits, st) : launch_variant_p<KF, VB, false>(a, tb, splits, st);
}

}  // namespace

int TQ_CAT(flash_mma_resident_ctas_, TQ_GEOM)() { return g_ctas_per_sm_seen; }
int TQ_CAT(flash_mma_ctas_per_sm_, TQ_GEOM)(const FlashArgs& a) {
  const bool v_affine = a.v_format == TQ_KV_AFFINE;
  const int vb = v_affine ? 40 : a.v_bits;
  const int kf = a.k_format == TQ_KV_AFFINE ? KF_AFFINE8
                 : a.k_format == TQ_KV_POLAR ? (a.k_bits == 3 ? KF_POLAR3 : KF_POLAR4) : KF_DENSE;
#define TQ_CTAS(K, V) if (kf == K && vb == V) return Layout<K, V>::ctas
  TQ_CTAS(KF_DENSE, 3); TQ_CTAS(KF_DENSE, 4); TQ_CTAS(KF_DENSE, 40);
  TQ_CTAS(KF_POLAR3, 3); TQ_CTAS(KF_POLAR3, 4); TQ_CTAS(KF_POLAR4, 3); TQ_CTAS(KF_POLAR4, 4);
  TQ_CTAS(KF_AFFINE8, 3); TQ_CTAS(KF_AFFINE8, 4); TQ_CTAS(KF_AFFINE8, 40);
#undef TQ_CTAS
  return 1;
}

int TQ_CAT(launch_flash_mma_, TQ_GEOM)(const FlashArgs& a, int splits, const MmaOutput& mo, cudaStream_t st) {
  MmaTables tb;
  memset(&tb, 0, sizeof(tb));
  tb.status = mo.status;
  tb.counters = mo.counters;
  tb.hints = mo.hints;
  tb.splits = splits;
  tb.out_mode = mo.out_mode;
  tb.out_dtype = mo.out_dtype;
  tb.out = mo.out;
  tb.out_batch_stride = mo.out_batch_stride;
  tb.out_head_stride = mo.out_head_stride;
  tb.om = mo.om;
  tb.ol = mo.ol;
  tb.oacc = mo.oacc;
  tb.n_peers = mo.n_peers;
  tb.peer_unordered = mo.peer_unordered;
  tb.g_m = mo.g_m;
  tb.g_l = mo.g_l;
  tb.g_acc = mo.g_acc;
  tb.g_stride = mo.g_stride;
  tb.g_flags = mo.g_flags;
  tb.g_ranks = mo.g_ranks;
  tb.g_expect = a.batch * a.n_kv_heads;
  tb.g_limit_ns = mo.g_limit_ns;
  for (int i = 0; i < 8; ++i) {
    tb.peer_m[i] = mo.peer_m[i];
    tb.peer_l[i] = mo.peer_l[i];
    tb.peer_acc[i] = mo.peer_acc[i];
    tb.peer_counter[i] = mo.peer_counter[i];
  }
  const bool v_affine = a.v_format == TQ_KV_AFFINE;
  if (v_affine) {
    for (int i = 0; i < 16; ++i) tb.v_c16[i] = (uint16_t)(i == 0 ? 0 : __half_as_ushort(__float2half_rn((float)i)));
    tb.v_post = 1.0f;
  } else {
    ScaledBook vb;
    scale_codebook(a.v_cent.v, 1 << a.v_bits, &vb);
    memcpy(tb.v_c16, vb.c16, sizeof(tb.v_c16));
    tb.v_post = 1.0f / vb.beta;
  }
  tb.k_post = a.attn_scale * kLog2e;
  int kf = KF_DENSE;
  if (a.k_format == TQ_KV_POLAR) {
    ScaledBook kb;
    scale_codebook(a.k_cent.v, 1 << a.k_bits, &kb);
    memcpy(tb.k_c16, kb.c16, sizeof(tb.k_c16));
    tb.k_post = a.attn_scale * kLog2e / ((float)kDim * kb.beta);
    kf = a.k_bits == 3 ? KF_POLAR3 : KF_POLAR4;
  }
  const bool k_bf16 = a.k_format == TQ_KV_DENSE && a.k_dtype == TQ_BF16;
  if (v_affine) {
    if (a.k_format == TQ_KV_AFFINE) return launch_variant<KF_AFFINE8, 40>(a, tb, splits, st);
    return k_bf16 ? launch_variant<KF_DENSE_BF16, 40>(a, tb, splits, st) : launch_variant<KF_DENSE, 40>(a, tb, splits, st);
  }
  if (a.k_format == TQ_KV_AFFINE)
    return a.v_bits == 3 ? launch_variant<KF_AFFINE8, 3>(a, tb, splits, st) : launch_variant<KF_AFFINE8, 4>(a, tb, splits, st);
  if (kf == KF_DENSE && k_bf16)
    return a.v_bits == 3 ? launch_variant<KF_DENSE_BF16, 3>(a, tb, splits, st) : launch_variant<KF_DENSE_BF16, 4>(a, tb, splits, st);
  if (kf == KF_DENSE) return a.v_bits == 3 ? launch_variant<KF_DENSE, 3>(a, tb, splits, st) : launch_variant<KF_DENSE, 4>(a, tb, splits, st);
  if (kf == KF_POLAR3) return a.v_bits == 3 ? launch_variant<KF_POLAR3, 3>(a, tb, splits, st) : launch_variant<KF_POLAR3, 4>(a, tb, splits, st);
  return a.v_bits == 3 ? launch_variant<KF_POLAR4, 3>(a, tb, splits, st) : launch_variant<KF_POLAR4, 4>(a, tb, splits, st);
}

}  // namespace tq
