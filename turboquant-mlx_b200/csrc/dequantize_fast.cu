// PolarQuant decode for head_dim 128 with TPV = 2 or 4 threads per vector.
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

template <typename T, int BITS, int TPV>
int launch_tpv(const FastDequantArgs& a, cudaStream_t st) {
  const int per_block = (32 / TPV) * kWarps;
  const int64_t groups = (a.n_vecs + per_block - 1) / per_block;
  const int64_t cap = (int64_t)num_sms() * 8;
  const int grid = (int)(groups < cap ? groups : cap);
  dequantize_split_kernel<T, BITS, TPV><<<grid, kWarps * 32, 0, st>>>(a);
  return check_launch("tq_dequantize (split per vector)");
}

template <typename T, int BITS>
int launch_fast(const FastDequantArgs& a, cudaStream_t st) {
  // 4 threads per vector measured fastest on B200 (2: 7 % slower).  A variant that looked codes up two
  // at a time in a lane-replicated float2 table executed 24 % fewer instructions and was no faster: the
  // two cross-thread stages (64 shuffles per thread) keep the shuffle / shared-memory pipe 65 % busy.
  return launch_tpv<T, BITS, 4>(a, st);
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
