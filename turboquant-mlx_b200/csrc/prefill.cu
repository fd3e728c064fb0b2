// tq_prefill_sdpa: causal (or full) scaled-dot-product attention over dense
// f16 / bf16 Q, K, V with head_dim 128 -- the prefill step that precedes the
// quantized decode path (the reference hands this to its array library's SDPA,
// turboquant_mlx/patch.py:37, on keys / values that update_and_fetch returned
// in the input dtype, cache.py:100-150).
//
// Blackwell-native formulation, one CTA per (128-query tile, query head, batch):
//   * Q, K and V tiles arrive by TMA (cp.async.bulk.tensor, 128-byte swizzle)
//     into shared memory; K / V tiles of 128 keys run through a 2-stage ring.
//   * S = Q K^T and O += P V are tcgen05.mma (cta_group::1, kind::f16, M = N =
//     128, K = 16 per instruction) issued by one thread.  Three score buffers
//     and O live in tensor memory (128 lanes x 128 fp32 columns each); P goes
//     over the upper half of its scores as packed 16-bit pairs and is the A
//     operand of the second product straight from tensor memory.  V is consumed
//     as stored (keys x head_dim, head_dim contiguous) through an MN-major
//     descriptor.
//   * Two groups of four warps (one thread per query row each) take the K/V tiles
//     in turn, group 0 the even ones and group 1 the odd ones: tcgen05.ld the
//     scores, online softmax in the log2 domain, tcgen05.st of P.  The running
//     row maximum travels from tile to tile through a shared-memory mailbox; a
//     group's exponentials (special-function unit) run while the other group
//     loads, masks and reduces its scores, and the tensor core works meanwhile
//     on the products of the surrounding tiles.  O is rescaled lazily (only when
//     a row maximum grows by more than 2^8) by the group that sees the growth.
//   * Every wait is bounded; a wait that gives up sets the status word, the CTA
//     drains its copies, frees its tensor memory and returns.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace tq {
namespace {

constexpr int kD = 128;          // head_dim
constexpr int kBM = 128;         // queries per CTA
constexpr int kBN = 128;         // keys per tile
constexpr int kKStages = 3;      // K tiles run three ahead of the softmax
constexpr int kVStages = 2;
constexpr int kSBufs = 3;        // score buffers in tensor memory: tile j uses buffer j % 3
constexpr int kGroupThreads = 128;               // one softmax group: one thread per query row
constexpr int kSoftmaxThreads = 2 * kGroupThreads;
constexpr int kThreads = kSoftmaxThreads + 64;   // + TMA warp + MMA warp
constexpr int kProducerWarp = kSoftmaxThreads / 32, kMmaWarp = kProducerWarp + 1;
constexpr uint32_t kTileBytes = kBM * kD * 2;    // 32 KiB: one 128 x 128 16-bit tile
constexpr uint32_t kHalfBytes = kTileBytes / 2;  // one 128-row x 64-element swizzle block
constexpr uint32_t kSpin = 1u << 20;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescale = 8.0f;                 // log2 units: P stays <= 2^8
// Tensor memory (512 columns x 128 lanes): scores of tile j at columns 128 (j % 3); its P (16-bit
// pairs, 64 columns for 128 keys) goes over columns 64..127 of the same buffer; O at 384.
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kColS = 0, kColO = 384, kColPinS = 64;

struct Smem {                    // offsets from the 1024-byte aligned base
  static constexpr uint32_t q = 0;
  static constexpr uint32_t k0 = q + kTileBytes;                   // K stage s: k0 + s * kTileBytes
  static constexpr uint32_t v0 = k0 + kKStages * kTileBytes;       // V stage s: v0 + s * kTileBytes
  static constexpr uint32_t mbox = v0 + kVStages * kTileBytes;     // running row maxima [2][128], then final (m, l) [2][2][128]
  static constexpr uint32_t bars = mbox + 6 * kBM * 4;
  static constexpr uint32_t tmem_slot = bars + 32 * 8;
  static constexpr uint32_t total = tmem_slot + 16;
};
constexpr uint32_t kSmemBytes = Smem::total + 1024;   // slack for the alignment

struct PrefillArgs {
  void* out;
  int64_t o_batch_stride, o_head_stride, o_row_stride;   // elements
  int seq_q, seq_k, n_rep, causal, bf16;
  float scale_log2;
  int* status;
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Bounded wait; gives up early once any wait of this launch has already failed.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, const int* status) {
  for (uint32_t it = 0; it < kSpin; ++it) {
    if (status && (it & 1023u) == 1023u && *reinterpret_cast<const volatile int*>(status) != 0) return false;
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
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, int c0, int c1, int c2, int c3,
                                            uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4, %5}], [%6];"
      ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "r"(bar)
      : "memory");
}
// Shared-memory matrix descriptor, 128-byte swizzle, 8-row groups 1024 bytes apart.
// K-major operands ignore the leading offset; MN-major ones use it as the distance
// between 64-element blocks along M / N.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t leading_bytes) {
  return (uint64_t)((addr >> 4) & 0x3FFFu) | ((uint64_t)((leading_bytes >> 4) & 0x3FFFu) << 16) |
         ((uint64_t)(1024u >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// A operand from tensor memory (row i in lane i, 16-bit elements packed two per column)
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
        "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
        "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]),
        "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
        "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
        "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
      ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
        "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
      : "memory");
}
__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack16(float a, float b, bool bf16) {
  if (bf16) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
  }
  const __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<const uint32_t*>(&h);
}

// Barrier slots (8 bytes each) inside Smem::bars.
enum : int { B_Q = 0, B_K_FULL = 1, B_K_EMPTY = 4, B_V_FULL = 7, B_V_EMPTY = 9, B_S_FULL = 11, B_P_FULL = 14,
             B_PV_DONE = 17 /* 2: by tile parity */, B_ALL_DONE = 19, B_MBOX = 20 /* 8: [row group][tile parity] */ };

__global__ void __launch_bounds__(kThreads, 1)
prefill_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const PrefillArgs a) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem = smem_raw + (sbase - smem_u32(smem_raw));
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q_tile = (int)gridDim.x - 1 - (int)blockIdx.x;     // longest (latest) tiles first
  const int head = blockIdx.y, batch = blockIdx.z;
  const int kv_head = head / a.n_rep;
  const int q0 = q_tile * kBM;
  const int off = a.seq_k - a.seq_q;                           // key index of query row 0's diagonal
  // keys this tile can see: [0, k_end)
  const int k_end = a.causal ? min(a.seq_k, q0 + kBM + off) : a.seq_k;
  const int n_tiles = (k_end + kBN - 1) / kBN;
  auto bar = [&](int i) { return sbase + Smem::bars + 8u * i; };
  auto wait = [&](uint32_t b, uint32_t parity) { return mbar_wait(b, parity, a.status); };

  if (tid == 0) {
    mbar_init(bar(B_Q), 1);
    for (int s = 0; s < kKStages; ++s) {
      mbar_init(bar(B_K_FULL + s), 1);
      mbar_init(bar(B_K_EMPTY + s), 1);
    }
    for (int s = 0; s < kVStages; ++s) {
      mbar_init(bar(B_V_FULL + s), 1);
      mbar_init(bar(B_V_EMPTY + s), 1);
    }
    for (int i = 0; i < kSBufs; ++i) {
      mbar_init(bar(B_S_FULL + i), 1);
      mbar_init(bar(B_P_FULL + i), kGroupThreads);
    }
    mbar_init(bar(B_PV_DONE), 1);
    mbar_init(bar(B_PV_DONE + 1), 1);
    mbar_init(bar(B_ALL_DONE), 1);
    for (int i = 0; i < 8; ++i) mbar_init(bar(B_MBOX + i), 32);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == kMmaWarp) {   // this warp owns the tensor-memory allocation
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(sbase + Smem::tmem_slot),
                 "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem = *reinterpret_cast<volatile uint32_t*>(smem + Smem::tmem_slot);
  const uint32_t tmem_o = tmem + kColO;

  if (warp == kProducerWarp) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      mbar_expect_tx(bar(B_Q), kTileBytes);
      tma_load_4d(sbase + Smem::q, &map_q, 0, q0, head, batch, bar(B_Q));
      tma_load_4d(sbase + Smem::q + kHalfBytes, &map_q, 64, q0, head, batch, bar(B_Q));
      auto load_k = [&](int j) {
        const int s = j % kKStages;
        if (j >= kKStages && !wait(bar(B_K_EMPTY + s), ((j / kKStages) - 1) & 1)) return false;
        const uint32_t dst = sbase + Smem::k0 + s * kTileBytes;
        mbar_expect_tx(bar(B_K_FULL + s), kTileBytes);
        tma_load_4d(dst, &map_k, 0, j * kBN, kv_head, batch, bar(B_K_FULL + s));
        tma_load_4d(dst + kHalfBytes, &map_k, 64, j * kBN, kv_head, batch, bar(B_K_FULL + s));
        return true;
      };
      auto load_v = [&](int j) {
        const int s = j % kVStages;
        if (j >= kVStages && !wait(bar(B_V_EMPTY + s), ((j / kVStages) - 1) & 1)) return false;
        const uint32_t dst = sbase + Smem::v0 + s * kTileBytes;
        mbar_expect_tx(bar(B_V_FULL + s), kTileBytes);
        tma_load_4d(dst, &map_v, 0, j * kBN, kv_head, batch, bar(B_V_FULL + s));
        tma_load_4d(dst + kHalfBytes, &map_v, 64, j * kBN, kv_head, batch, bar(B_V_FULL + s));
        return true;
      };
      // K runs ahead of V: the scores are computed up to three tiles ahead of the softmax
      int jk = 0, jv = 0;
      bool ok = true;
      while (ok && (jk < n_tiles || jv < n_tiles)) {
        if (jk < n_tiles && jk <= jv + 2) {
          ok = load_k(jk);
          if (ok) ++jk;
        } else {
          ok = load_v(jv);
          if (ok) ++jv;
        }
      }
      if (!ok) atomicExch(a.status, 11);
      // drain: every copy this thread issued has landed before the CTA may exit
      mbar_wait(bar(B_Q), 0, nullptr);
      for (int j = max(0, jk - kKStages); j < jk; ++j) mbar_wait(bar(B_K_FULL + j % kKStages), (j / kKStages) & 1, nullptr);
      for (int j = max(0, jv - kVStages); j < jv; ++j) mbar_wait(bar(B_V_FULL + j % kVStages), (j / kVStages) & 1, nullptr);
    }
  } else if (warp == kMmaWarp) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      const uint32_t fmt = a.bf16 ? 1u : 0u;
      // D f32, A / B f16 or bf16, M = 128, N = 128; B of the second product is MN-major
      const uint32_t idesc_qk = (1u << 4) | (fmt << 7) | (fmt << 10) | ((uint32_t)(kBN >> 3) << 17) |
                                ((uint32_t)(kBM >> 4) << 24);
      const uint32_t idesc_pv = idesc_qk | (1u << 16);
      bool ok = wait(bar(B_Q), 0);
      int fail = ok ? 0 : 12;
      // descriptors are built once; inside the loops only the 16-byte-unit address field moves
      uint64_t q_desc[kD / 16];
#pragma unroll
      for (int kk = 0; kk < kD / 16; ++kk)
        q_desc[kk] = smem_desc(sbase + Smem::q + (kk >> 2) * kHalfBytes + (kk & 3) * 32, 16);
      const uint64_t k_desc0 = smem_desc(sbase + Smem::k0, 16), v_desc0 = smem_desc(sbase + Smem::v0, kHalfBytes);
      auto issue_qk = [&](int j) {     // S[j % 3] = Q K_j^T
        const int s = j % kKStages;
        if (!wait(bar(B_K_FULL + s), (j / kKStages) & 1)) return false;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t kd = k_desc0 + (uint64_t)(s * (kTileBytes >> 4));
        const uint32_t d_tmem = tmem + kColS + (j % kSBufs) * kBN;
#pragma unroll
        for (int kk = 0; kk < kD / 16; ++kk)
          umma_f16(d_tmem, q_desc[kk], kd + (uint64_t)(((kk >> 2) * kHalfBytes + (kk & 3) * 32) >> 4), idesc_qk, kk > 0);
        umma_commit(bar(B_K_EMPTY + s));
        umma_commit(bar(B_S_FULL + j % kSBufs));
        return true;
      };
      for (int j = 0; j < kSBufs && j < n_tiles && ok; ++j)
        if (!issue_qk(j)) {
          ok = false;
          fail = 13;
        }
      for (int j = 0; j < n_tiles && ok; ++j) {
        const int s = j % kVStages;
        if (!wait(bar(B_V_FULL + s), (j / kVStages) & 1) || !wait(bar(B_P_FULL + j % kSBufs), (j / kSBufs) & 1)) {
          ok = false;
          fail = 14;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t vd = v_desc0 + (uint64_t)(s * (kTileBytes >> 4));
        const uint32_t p_tmem = tmem + kColS + (j % kSBufs) * kBN + kColPinS;
#pragma unroll
        for (int kk = 0; kk < kBN / 16; ++kk)    // 16 keys = 8 packed columns of P, 2 x 1024 bytes of V
          umma_f16_ts(tmem_o, p_tmem + kk * 8, vd + (uint64_t)(kk * (2048 >> 4)), idesc_pv,
                      (j > 0 || kk > 0) ? 1u : 0u);
        umma_commit(bar(B_V_EMPTY + s));
        umma_commit(bar(B_PV_DONE + (j & 1)));
        // the scores three tiles on go over this tile's buffer: the tensor core runs its work in
        // issue order, so they follow the product that has just read P from it
        if (j + kSBufs < n_tiles && !issue_qk(j + kSBufs)) {
          ok = false;
          fail = 13;
          break;
        }
      }
      umma_commit(bar(B_ALL_DONE));
      if (fail) atomicExch(a.status, fail);
    }
  } else {
    // ---------------- softmax: group `who` takes the tiles j = who, who + 2, ...; one row per thread ----------------
    const int who = warp >> 2, rg = warp & 3;
    const int row = rg * 32 + lane;                        // = tensor-memory lane
    const uint32_t lane_base = (uint32_t)(rg * 32) << 16;
    float* mbox = reinterpret_cast<float*>(smem + Smem::mbox);    // [tile parity][row]
    float* fin = mbox + 2 * kBM;                                  // [m | l][who][row]
    const int kmax = a.causal ? q0 + row + off : a.seq_k - 1;     // last key this row may see
    float m_mine = -INFINITY, l_mine = 0.f;                       // l_mine is relative to m_mine
    bool ok = true;
    // the 64 scores of one half row: load, mask what the row may not see
    auto load_half = [&](int j, int h, uint32_t (&v)[2][32]) {
      const uint32_t src = tmem + kColS + (j % kSBufs) * kBN + lane_base + h * 64;
      tmem_ld32(src, v[0]);
      tmem_ld32(src + 32, v[1]);
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      const bool need_mask = (j * kBN + kBN - 1 > (a.causal ? q0 + off : a.seq_k - 1)) || (j * kBN + kBN > a.seq_k);
      if (need_mask) {
        const int klim = min(kmax, a.seq_k - 1) - (j * kBN + h * 64);     // columns <= klim are visible
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i > klim) v[c][i] = 0xff800000u;   // -inf
      }
    };
    auto half_max = [&](const uint32_t (&v)[2][32]) {
      float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four independent chains
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 32; ++i) mx[i & 3] = fmaxf(mx[i & 3], __uint_as_float(v[c][i]));
      return fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
    };
    // exponentials of a half row -> 32 packed columns of P at `dst`; returns their sum
    auto half_exp = [&](const uint32_t (&v)[2][32], float neg_m, uint32_t dst) {
      uint32_t pk[32];
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c = 0; c < 2; ++c)
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = ex2(fmaf(__uint_as_float(v[c][2 * i]), a.scale_log2, neg_m));
          const float p1 = ex2(fmaf(__uint_as_float(v[c][2 * i + 1]), a.scale_log2, neg_m));
          ls[i & 3] += p0 + p1;
          pk[c * 16 + i] = pack16(p0, p1, a.bf16);
        }
      tmem_st32(dst, pk);
      return (ls[0] + ls[1]) + (ls[2] + ls[3]);
    };
    for (int j = who; j < n_tiles && ok; j += 2) {
      if (!__all_sync(0xffffffffu, wait(bar(B_S_FULL + j % kSBufs), (j / kSBufs) & 1))) {   // warp-uniform: aligned tcgen05 ops follow
        if (lane == 0) atomicExch(a.status, 15);
        ok = false;
        break;
      }
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      // pass 1: the row maximum (the lower half is read again for its exponentials; the upper half stays)
      uint32_t sv[2][32];
      load_half(j, 0, sv);
      float mraw = half_max(sv);
      load_half(j, 1, sv);
      mraw = fmaxf(mraw, half_max(sv));
      const float mt = mraw * a.scale_log2;              // scale > 0: order preserved
      // the running maximum after the previous tile comes from the other group
      if (j > 0) {
        if (!__all_sync(0xffffffffu, wait(bar(B_MBOX + rg * 2 + ((j - 1) & 1)), ((j - 1) >> 1) & 1))) {
          if (lane == 0) atomicExch(a.status, 18);
          ok = false;
          break;
        }
        const float m_prev = mbox[((j - 1) & 1) * kBM + row];
        if (m_prev != m_mine) {
          l_mine *= m_mine == -INFINITY ? 0.f : ex2(m_mine - m_prev);
          m_mine = m_prev;
        }
      }
      // lazy rescale: the reference maximum only moves when a row maximum outgrows it by 2^8
      const bool grow = mt > m_mine + kRescale;
      float alpha = 1.f;
      if (grow) {
        alpha = m_mine == -INFINITY ? 0.f : ex2(m_mine - mt);
        m_mine = mt;
        l_mine *= alpha;
      }
      // publish before touching O: the other group only scales its P with it, and its product is
      // issued after this tile's, which waits for the arrival at the end of this iteration
      mbox[(j & 1) * kBM + row] = m_mine;
      mbar_arrive(bar(B_MBOX + rg * 2 + (j & 1)));
      if (j > 0 && __any_sync(0xffffffffu, grow)) {
        // O must be complete up to the previous tile before it is rescaled
        if (!__all_sync(0xffffffffu, wait(bar(B_PV_DONE + ((j - 1) & 1)), ((j - 1) >> 1) & 1))) {
          if (lane == 0) atomicExch(a.status, 16);
          ok = false;
          break;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {      // rare path: kept small in registers
          uint32_t ov[16];
          tmem_ld16(tmem_o + lane_base + c * 16, ov);
          asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
          for (int i = 0; i < 16; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
          tmem_st16(tmem_o + lane_base + c * 16, ov);
        }
      }
      if (j == 1) {
        // start half a period behind group 0, so that one group's exponentials run while the other
        // loads and reduces scores
        if (!__all_sync(0xffffffffu, wait(bar(B_P_FULL), 0))) {
          if (lane == 0) atomicExch(a.status, 19);
          ok = false;
          break;
        }
      }
      // pass 2: P over columns 64..127 of the scores (both halves of which are in registers or consumed by now)
      const float neg_m = m_mine == -INFINITY ? 0.f : -m_mine;
      const uint32_t p_dst = tmem + kColS + (j % kSBufs) * kBN + lane_base + kColPinS;
      l_mine += half_exp(sv, neg_m, p_dst + 32);          // keys 64..127 -> packed columns 32..63
      load_half(j, 0, sv);
      l_mine += half_exp(sv, neg_m, p_dst);               // keys 0..63 -> packed columns 0..31
      asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      mbar_arrive(bar(B_P_FULL + j % kSBufs));
    }
    if (ok && n_tiles > 0) {
      if (!__all_sync(0xffffffffu, wait(bar(B_ALL_DONE), 0))) {
        if (lane == 0) atomicExch(a.status, 17);
        ok = false;
      }
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    // the two groups combine their row sums (each relative to its own last maximum); group 0 writes
    // output columns 0..63, group 1 columns 64..127
    fin[who * kBM + row] = m_mine;
    fin[(2 + who) * kBM + row] = l_mine;
    asm volatile("bar.sync %0, 64;" ::"r"(1 + rg) : "memory");
    const float m_oth = fin[(who ^ 1) * kBM + row], l_oth = fin[(2 + (who ^ 1)) * kBM + row];
    const float m_fin = fmaxf(m_mine, m_oth);
    const float l_row = (m_mine == -INFINITY ? 0.f : l_mine * ex2(m_mine - m_fin)) +
                        (m_oth == -INFINITY ? 0.f : l_oth * ex2(m_oth - m_fin));
    if (ok && n_tiles > 0) {
      const float inv = l_row > 0.f ? 1.f / l_row : 0.f;
      const bool live = q0 + row < a.seq_q;
      uint8_t* orow = reinterpret_cast<uint8_t*>(a.out) + who * 128 +
                      2 * (batch * a.o_batch_stride + head * a.o_head_stride + (int64_t)(q0 + row) * a.o_row_stride);
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t ov[32];
        tmem_ld32(tmem_o + lane_base + who * 64 + c * 32, ov);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (live) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 w;
            w.x = pack16(__uint_as_float(ov[8 * i]) * inv, __uint_as_float(ov[8 * i + 1]) * inv, a.bf16);
            w.y = pack16(__uint_as_float(ov[8 * i + 2]) * inv, __uint_as_float(ov[8 * i + 3]) * inv, a.bf16);
            w.z = pack16(__uint_as_float(ov[8 * i + 4]) * inv, __uint_as_float(ov[8 * i + 5]) * inv, a.bf16);
            w.w = pack16(__uint_as_float(ov[8 * i + 6]) * inv, __uint_as_float(ov[8 * i + 7]) * inv, a.bf16);
            *reinterpret_cast<uint4*>(orow + c * 64 + i * 16) = w;
          }
        }
      }
    }
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (warp == kMmaWarp) {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
  }
}

// ---- host side: tensor maps ------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// (batch, heads, rows, 128) tensor with arbitrary (16-byte multiple) strides; box = 64 elements x 128 rows
int make_map(CUtensorMap* map, const void* base, int bf16, int64_t batch, int64_t heads, int64_t rows,
             int64_t batch_stride, int64_t head_stride, int64_t row_stride) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return set_error(TQ_ERR_LAUNCH, "cuTensorMapEncodeTiled is not available from this driver");
  const cuuint64_t dims[4] = {(cuuint64_t)kD, (cuuint64_t)rows, (cuuint64_t)heads, (cuuint64_t)batch};
  // a stride of a size-1 dimension is never used for addressing: give the encoder the packed value
  if (heads == 1) head_stride = rows * row_stride;
  if (batch == 1) batch_stride = heads * head_stride;
  const cuuint64_t strides[3] = {(cuuint64_t)row_stride * 2, (cuuint64_t)head_stride * 2, (cuuint64_t)batch_stride * 2};
  const cuuint32_t box[4] = {64, (cuuint32_t)kBM, 1, 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  const CUresult r = fn(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4,
                        const_cast<void*>(base), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                        CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return set_error(TQ_ERR_LAUNCH, "cuTensorMapEncodeTiled failed with code %d", (int)r);
  return TQ_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace
}  // namespace tq

extern "C" int tq_prefill_sdpa(const void* q, const void* k, const void* v, void* out, int dtype, int batch,
                               int n_q_heads, int n_kv_heads, int64_t seq_q, int64_t seq_k, int dim,
                               int64_t q_batch_stride, int64_t q_head_stride, int64_t q_row_stride,
                               int64_t k_batch_stride, int64_t k_head_stride, int64_t k_row_stride,
                               int64_t v_batch_stride, int64_t v_head_stride, int64_t v_row_stride,
                               int64_t o_batch_stride, int64_t o_head_stride, int64_t o_row_stride,
                               float attn_scale, int causal, int* status, void* stream) {
  using namespace tq;
  TQ_REQUIRE(q && k && v && out && status, TQ_ERR_BAD_ARG, "tq_prefill_sdpa: NULL pointer");
  TQ_REQUIRE(dim == kD, TQ_ERR_BAD_DIM, "tq_prefill_sdpa supports head_dim 128, got %d", dim);
  TQ_REQUIRE(dtype == TQ_F16 || dtype == TQ_BF16, TQ_ERR_UNSUPPORTED, "tq_prefill_sdpa takes f16 or bf16 tensors");
  TQ_REQUIRE(batch > 0 && n_q_heads > 0 && n_kv_heads > 0 && seq_q > 0 && seq_k > 0, TQ_ERR_BAD_ARG,
             "batch, head counts and sequence lengths must be positive");
  TQ_REQUIRE(n_q_heads % n_kv_heads == 0, TQ_ERR_HEAD_MISMATCH, "n_q_heads (%d) must equal n_kv_heads (%d) * n_rep",
             n_q_heads, n_kv_heads);
  TQ_REQUIRE(!causal || seq_k >= seq_q, TQ_ERR_BAD_ARG, "causal attention needs seq_k >= seq_q");
  TQ_REQUIRE(attn_scale > 0.f, TQ_ERR_BAD_ARG, "attn_scale must be positive, got %g", (double)attn_scale);
  TQ_REQUIRE(seq_k < (1ll << 31) - 256 && seq_q < (1ll << 31) - 256 && batch <= 65535 && n_q_heads <= 65535,
             TQ_ERR_BAD_ARG, "shape out of range");
  const int64_t strides[] = {q_batch_stride, q_head_stride, q_row_stride, k_batch_stride, k_head_stride, k_row_stride,
                             v_batch_stride, v_head_stride, v_row_stride, o_batch_stride, o_head_stride, o_row_stride};
  for (int64_t s : strides)
    TQ_REQUIRE(s >= 0 && s % 8 == 0, TQ_ERR_MISALIGNED, "tq_prefill_sdpa: strides must be multiples of 8 elements");
  TQ_REQUIRE(aligned16(q) && aligned16(k) && aligned16(v) && aligned16(out), TQ_ERR_MISALIGNED,
             "tq_prefill_sdpa: tensors must be 16-byte aligned");
  const int bf16 = dtype == TQ_BF16;
  CUtensorMap mq, mk, mv;
  int rc;
  if ((rc = make_map(&mq, q, bf16, batch, n_q_heads, seq_q, q_batch_stride, q_head_stride, q_row_stride))) return rc;
  if ((rc = make_map(&mk, k, bf16, batch, n_kv_heads, seq_k, k_batch_stride, k_head_stride, k_row_stride))) return rc;
  if ((rc = make_map(&mv, v, bf16, batch, n_kv_heads, seq_k, v_batch_stride, v_head_stride, v_row_stride))) return rc;
  PrefillArgs a;
  a.out = out;
  a.o_batch_stride = o_batch_stride;
  a.o_head_stride = o_head_stride;
  a.o_row_stride = o_row_stride;
  a.seq_q = (int)seq_q;
  a.seq_k = (int)seq_k;
  a.n_rep = n_q_heads / n_kv_heads;
  a.causal = causal ? 1 : 0;
  a.bf16 = bf16;
  a.scale_log2 = attn_scale * kLog2e;
  a.status = status;
  static std::once_flag once;
  static cudaError_t attr_err = cudaSuccess;
  std::call_once(once, [] {
    attr_err = cudaFuncSetAttribute(prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
  });
  if (attr_err != cudaSuccess) return set_error(TQ_ERR_LAUNCH, "tq_prefill_sdpa: %s", cudaGetErrorString(attr_err));
  const dim3 grid((unsigned)((seq_q + kBM - 1) / kBM), (unsigned)n_q_heads, (unsigned)batch);
  prefill_kernel<<<grid, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(mq, mk, mv, a);
  return check_launch("tq_prefill_sdpa");
}
