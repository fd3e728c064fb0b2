// PolarQuant decode for head_dim 128 with TPV = 2 or 4 threads per vector (4-bit rows) and the
// pair-table kernel for 3-bit rows (dequantize_pairs_kernel below).
//
// Thread q of a group reconstructs elements [EPT q, EPT q + EPT), EPT = 128 / TPV:
// codes -> centroid * s through a small shared-memory table, log2(EPT) butterfly
// stages in registers and log2(TPV) through shuffles (same pairs, same order as
// the general kernel, so float32 results are bit-identical), then
// ((bfly * s) * sign) * norm and the cast to the output type.
// 3-bit rows are first compacted from thirteen 30-bit words into a dense 384-bit
// string so that every code sits at a compile-time bit position; the thread then
// selects its part of the string by q with register selects (no divergence).
// Requirements (checked by the launcher): dim 128, bits 3 or 4, contiguous
// output rows, 16-byte aligned output.

#include <type_traits>

#include "common.cuh"

namespace tq {
namespace {

constexpr int kDimF = 128;
constexpr int kWarps = 8;

struct FastDequantArgs {
  const uint32_t* packed;
  int64_t packed_outer_stride;
  const float* norms;
  int64_t norms_outer_stride;
  int64_t n_vecs;
  uint32_t n_inner;
  void* out;
  SignMask signs;
  Table16 cs;       // centroid * s
  float s;
};

template <typename T, int BITS, int TPV>
__global__ void __launch_bounds__(kWarps * 32)
dequantize_split_kernel(const FastDequantArgs a) {
  constexpr int EPT = kDimF / TPV;
  constexpr int VPWARP = 32 / TPV;
  constexpr int PDIM = packed_words(kDimF, BITS);
  constexpr int DW = EPT * BITS / 32;           // dense words per thread
  __shared__ float cs_s[16];
  if (threadIdx.x < 16) cs_s[threadIdx.x] = a.cs.v[threadIdx.x];
  __syncthreads();
  const uint32_t cs_addr = (uint32_t)__cvta_generic_to_shared(cs_s);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int q = lane % TPV, vs = lane / TPV;
  const int64_t wg = (int64_t)blockIdx.x * kWarps + warp;
  const int64_t wstride = (int64_t)gridDim.x * kWarps;

  for (int64_t vb = wg * VPWARP; vb < a.n_vecs; vb += wstride * VPWARP) {
    const int64_t v = vb + vs;
    const bool valid = v < a.n_vecs;
    const int64_t vl = valid ? v : a.n_vecs - 1;
    const uint32_t o_idx = (uint32_t)vl / a.n_inner, i_idx = (uint32_t)vl - o_idx * a.n_inner;
    const uint32_t* prow = a.packed + (int64_t)o_idx * a.packed_outer_stride + (int64_t)i_idx * PDIM;
    const float nrm = __ldg(a.norms + (int64_t)o_idx * a.norms_outer_stride + i_idx);

    uint32_t dense[DW + 1];
    if (BITS == 4) {
#pragma unroll
      for (int w = 0; w < DW; ++w) dense[w] = __ldg(prow + DW * q + w);
      dense[DW] = 0;
    } else {
      // thirteen 30-bit words -> twelve dense words (every thread of the group does the same)
      uint32_t W[13];
#pragma unroll
      for (int w = 0; w < 13; ++w) W[w] = __ldg(prow + w);
      uint32_t D[13];
#pragma unroll
      for (int k = 0; k < 12; ++k) {
        const int bit = 32 * k, w = bit / 30, off = bit % 30;          // dense word k starts in word w
        uint32_t d = W[w] >> off;                                        // 30 - off bits
        if (w + 1 < 13) d |= W[w + 1] << (30 - off);
        if (60 - off < 32 && w + 2 < 13) d |= W[w + 2] << (60 - off);
        D[k] = d;
      }
      D[12] = 0;
#pragma unroll
      for (int w = 0; w <= DW; ++w) {
        uint32_t sel = D[w];                                             // q == 0
#pragma unroll
        for (int qq = 1; qq < TPV; ++qq) sel = (q == qq) ? D[(qq * DW + w) < 13 ? (qq * DW + w) : 12] : sel;
        dense[w] = sel;
      }
    }
    float y[EPT];
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
      const int bit = i * BITS, w = bit >> 5, sh = bit & 31;
      uint32_t c;
      if (sh + BITS <= 32) c = dense[w] >> sh;
      else c = __funnelshift_r(dense[w], dense[w + 1], sh);
      float val;
      const uint32_t addr = cs_addr + ((c & ((1u << BITS) - 1u)) << 2);
      asm volatile("ld.shared.f32 %0, [%1];" : "=f"(val) : "r"(addr));
      y[i] = val;
    }
#pragma unroll
    for (int h = 1; h < EPT; h <<= 1) {
#pragma unroll
      for (int j = 0; j < EPT; ++j) {
        if ((j & h) == 0) {
          const float p = y[j], r = y[j + h];
          y[j] = __fadd_rn(p, r);
          y[j + h] = __fsub_rn(p, r);
        }
      }
    }
#pragma unroll
    for (int k = 1; k < TPV; k <<= 1) {
      const float sg = (q & k) ? -1.0f : 1.0f;   // upper partner: o - y = fma(y, -1, o), rounded like the subtraction
#pragma unroll
      for (int j = 0; j < EPT; ++j) y[j] = __fmaf_rn(y[j], sg, __shfl_xor_sync(0xffffffffu, y[j], k));
    }
    // ((bfly * s) * sign) * norm, left to right as the reference writes it
    T* orow = reinterpret_cast<T*>(a.out) + vl * kDimF + q * EPT;
    if (std::is_same<T, float>::value) {
#pragma unroll
      for (int i = 0; i < EPT; i += 4) {
        float4 r;
        float* rp = &r.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float t = __fmul_rn(y[i + k], a.s);
          rp[k] = __fmul_rn(__uint_as_float(__float_as_uint(t) ^ sign_bit_at(a.signs, EPT * q + i + k)), nrm);
        }
        if (valid) *reinterpret_cast<float4*>(reinterpret_cast<float*>(orow) + i) = r;
      }
    } else {
#pragma unroll
      for (int i = 0; i < EPT; i += 8) {
        uint32_t pk[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float r2[2];
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const float t = __fmul_rn(y[i + 2 * k + e], a.s);
            r2[e] = __fmul_rn(__uint_as_float(__float_as_uint(t) ^ sign_bit_at(a.signs, EPT * q + i + 2 * k + e)), nrm);
          }
          if (std::is_same<T, __half>::value) {
            const __half2 h = __floats2half2_rn(r2[0], r2[1]);
            pk[k] = *reinterpret_cast<const uint32_t*>(&h);
          } else {
            const __nv_bfloat162 h = __floats2bfloat162_rn(r2[0], r2[1]);
            pk[k] = *reinterpret_cast<const uint32_t*>(&h);
          }
        }
        if (valid) *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(orow) + i) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
    }
  }
}

// 3-bit rows, 4 threads per vector: codes two at a time through a lane-replicated pair table.
//
// Thread q of a vector's group owns elements [32 q, 32 q + 32).  Their codes lie in the four 30-bit
// words 3 q .. 3 q + 3 of the row, starting 2 q codes into the first one: the thread loads those four
// words, closes the 2-bit gaps (120 dense bits) and shifts by 6 q, after which every code pair sits at
// a compile-time position.  A pair (6 bits) indexes a table of float2 (centroid * s of both codes)
// replicated per lane (entry * 256 + lane * 8 bytes: conflict free), so a lookup is one shift, one
// logic op and one 8-byte shared load for two elements.  The two cross-thread butterfly stages use
// fma(y, +-1, partner), which rounds exactly like the add / subtract it replaces; for 16-bit outputs
// the sign vector is applied to the packed pair (the flip commutes with every rounding step).
template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
dequantize_pairs_kernel(const FastDequantArgs a) {
  constexpr int TPV = 4, EPT = 32, VPWARP = 8, PDIM = 13;
  __shared__ __align__(16) float2 pair_s[64 * 32];
  for (int i = threadIdx.x; i < 64 * 32; i += kWarps * 32) {
    const int e = i >> 5;
    pair_s[i] = make_float2(a.cs.v[e & 7], a.cs.v[e >> 3]);
  }
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int q = lane % TPV, vs = lane / TPV;
  const uint32_t lut = (uint32_t)__cvta_generic_to_shared(pair_s) + lane * 8;
  const uint32_t sw = a.signs.w[q];                 // signs of this thread's 32 elements
  uint32_t pm[16];                                  // 16-bit outputs: sign bits of an element pair at bits 15 and 31
#pragma unroll
  for (int j = 0; j < 16; ++j) pm[j] = (((sw >> (2 * j)) & 1u) << 15) | (((sw >> (2 * j + 1)) & 1u) << 31);
  const float sg1 = (q & 1) ? -1.0f : 1.0f, sg2 = (q & 2) ? -1.0f : 1.0f;
  const int sh = 6 * q;
  const int64_t wg = (int64_t)blockIdx.x * kWarps + warp;
  const int64_t wstride = (int64_t)gridDim.x * kWarps;

  for (int64_t vb = wg * VPWARP; vb < a.n_vecs; vb += wstride * VPWARP) {
    const int64_t v = vb + vs;
    const bool valid = v < a.n_vecs;
    const int64_t vl = valid ? v : a.n_vecs - 1;
    const uint32_t o_idx = (uint32_t)vl / a.n_inner, i_idx = (uint32_t)vl - o_idx * a.n_inner;
    const uint32_t* prow = a.packed + (int64_t)o_idx * a.packed_outer_stride + (int64_t)i_idx * PDIM + 3 * q;
    const float nrm = __ldg(a.norms + (int64_t)o_idx * a.norms_outer_stride + i_idx);
    const uint32_t w0 = __ldg(prow), w1 = __ldg(prow + 1), w2 = __ldg(prow + 2), w3 = __ldg(prow + 3);
    // four 30-bit words -> 120 dense bits, then this thread's 96 bits from bit 6 q on
    const uint32_t d0 = w0 | (w1 << 30), d1 = (w1 >> 2) | (w2 << 28), d2 = (w2 >> 4) | (w3 << 26), d3 = w3 >> 6;
    uint32_t dense[3];
    dense[0] = __funnelshift_r(d0, d1, sh);
    dense[1] = __funnelshift_r(d1, d2, sh);
    dense[2] = __funnelshift_r(d2, d3, sh);
    float y[EPT];
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const int bit = 6 * j, w = bit >> 5, s = bit & 31;
      uint32_t c;                                   // pair index * 256
      if (s + 6 <= 32) c = s >= 8 ? (dense[w] >> (s - 8)) : (dense[w] << (8 - s));
      else c = __funnelshift_r(dense[w], dense[w + 1], s) << 8;
      const uint32_t addr = lut + (c & 0x3F00u);
      float lo, hi;
      asm volatile("ld.shared.v2.f32 {%0, %1}, [%2];" : "=f"(lo), "=f"(hi) : "r"(addr));
      y[2 * j] = lo;
      y[2 * j + 1] = hi;
    }
#pragma unroll
    for (int h = 1; h < EPT; h <<= 1) {
#pragma unroll
      for (int j = 0; j < EPT; ++j) {
        if ((j & h) == 0) {
          const float p = y[j], r = y[j + h];
          y[j] = __fadd_rn(p, r);
          y[j + h] = __fsub_rn(p, r);
        }
      }
    }
    // partners 1 and 2: lower thread p + r, upper thread o - y = fma(y, -1, o)
#pragma unroll
    for (int j = 0; j < EPT; ++j) y[j] = __fmaf_rn(y[j], sg1, __shfl_xor_sync(0xffffffffu, y[j], 1));
#pragma unroll
    for (int j = 0; j < EPT; ++j) y[j] = __fmaf_rn(y[j], sg2, __shfl_xor_sync(0xffffffffu, y[j], 2));
    // ((bfly * s) * sign) * norm, left to right as the reference writes it
    T* orow = reinterpret_cast<T*>(a.out) + vl * kDimF + q * EPT;
    if (std::is_same<T, float>::value) {
#pragma unroll
      for (int i = 0; i < EPT; i += 4) {
        float4 r;
        float* rp = &r.x;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float t = __fmul_rn(y[i + k], a.s);
          rp[k] = __fmul_rn(__uint_as_float(__float_as_uint(t) ^ (((sw >> (i + k)) & 1u) << 31)), nrm);
        }
        if (valid) *reinterpret_cast<float4*>(reinterpret_cast<float*>(orow) + i) = r;
      }
    } else {
#pragma unroll
      for (int i = 0; i < EPT; i += 8) {
        uint32_t pk[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float r0 = __fmul_rn(__fmul_rn(y[i + 2 * k], a.s), nrm);
          const float r1 = __fmul_rn(__fmul_rn(y[i + 2 * k + 1], a.s), nrm);
          uint32_t bits;
          if (std::is_same<T, __half>::value) {
            const __half2 h = __floats2half2_rn(r0, r1);
            bits = *reinterpret_cast<const uint32_t*>(&h);
          } else {
            const __nv_bfloat162 h = __floats2bfloat162_rn(r0, r1);
            bits = *reinterpret_cast<const uint32_t*>(&h);
          }
          pk[k] = bits ^ pm[(i >> 1) + k];          // sign flip of the rounded pair = rounding of the flipped pair
        }
        if (valid) *reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(orow) + i) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
      }
    }
  }
}

template <typename T, int BITS, int TPV>
int launch_tpv(const FastDequantArgs& a, cudaStream_t st) {
  const int per_block = (32 / TPV) * kWarps;
  const int64_t groups = (a.n_vecs + per_block - 1) / per_block;
  const int64_t cap = (int64_t)num_sms() * 8;
  const int grid = (int)(groups < cap ? groups : cap);
  dequantize_split_kernel<T, BITS, TPV><<<grid, kWarps * 32, 0, st>>>(a);
  return check_launch("tq_dequantize (split per vector)");
}

template <typename T>
int launch_pairs(const FastDequantArgs& a, cudaStream_t st) {
  const int per_block = 8 * kWarps;
  const int64_t groups = (a.n_vecs + per_block - 1) / per_block;
  const int64_t cap = (int64_t)num_sms() * 8;
  const int grid = (int)(groups < cap ? groups : cap);
  dequantize_pairs_kernel<T><<<grid, kWarps * 32, 0, st>>>(a);
  return check_launch("tq_dequantize (pair table)");
}

template <typename T, int BITS>
int launch_fast(const FastDequantArgs& a, cudaStream_t st) {
  if (BITS == 3) return launch_pairs<T>(a, st);
  return launch_tpv<T, BITS, 4>(a, st);   // 4 threads per vector measured fastest on B200 (2: 7 % slower)
}

}  // namespace

// Returns TQ_ERR_UNSUPPORTED when the arguments do not qualify (caller falls back).
int try_launch_dequantize_fast(const uint32_t* packed, int64_t packed_outer_stride, const float* norms,
                               int64_t norms_outer_stride, int64_t n_outer, int64_t n_inner, int dim,
                               int bits, const Table16& cs, float s, const SignMask& signs, void* out,
                               int out_dtype, int64_t out_outer_stride, cudaStream_t st) {
  if (dim != kDimF || (bits != 3 && bits != 4)) return TQ_ERR_UNSUPPORTED;
  if (out_outer_stride != n_inner * dim) return TQ_ERR_UNSUPPORTED;          // output rows must be contiguous
  if ((reinterpret_cast<uintptr_t>(out) & 15u) != 0) return TQ_ERR_UNSUPPORTED;
  const int64_t n_vecs = n_outer * n_inner;
  if (n_vecs < 1024 || n_vecs >= (1LL << 31) || n_inner >= (1LL << 31)) return TQ_ERR_UNSUPPORTED;
  FastDequantArgs a;
  a.packed = packed;
  a.packed_outer_stride = packed_outer_stride;
  a.norms = norms;
  a.norms_outer_stride = norms_outer_stride;
  a.n_vecs = n_vecs;
  a.n_inner = (uint32_t)n_inner;
  a.out = out;
  a.signs = signs;
  a.cs = cs;
  a.s = s;
#define TQ_FAST(T) return bits == 3 ? launch_fast<T, 3>(a, st) : launch_fast<T, 4>(a, st)
  switch (out_dtype) {
    case TQ_F32: TQ_FAST(float);
    case TQ_F16: TQ_FAST(__half);
    case TQ_BF16: TQ_FAST(__nv_bfloat16);
    default: return TQ_ERR_UNSUPPORTED;
  }
#undef TQ_FAST
}

}  // namespace tq
