// PolarQuant encode of ONE vector by ONE warp (reference
// turboquant_mlx/quantizer.py:75-106 + packing.py:26-56): the body shared by the
// general quantize kernel and by the decode kernel's in-launch cache append, so
// that both produce the same words.
//
// Lane l holds elements [EPL*l, EPL*l + EPL).  Every float32 step that feeds the
// index compare uses an explicit round-to-nearest intrinsic (no contraction):
//   sum of squares : pairwise tree in natural index order (in-lane, then lanes 1, 2, 4, 8, 16 apart)
//   normalise      : x / max(sqrt(ss), 1e-8), IEEE division
//   rotate         : sign flip, raw Walsh-Hadamard butterfly
//   index          : number of thresholds exceeded (strict compare on the raw butterfly output)
//   pack           : element j -> word j / vpw, bit (j % vpw) * bits
#pragma once

#include "common.cuh"

namespace tq {

// x: this lane's EPL elements as float32.  idx_s: DIM bytes of shared memory owned by
// the calling warp.  Writes packed_words(DIM, BITS) words at prow and the norm at *norm_out.
template <int EPL, int BITS>
__device__ __forceinline__ void quantize_row_warp(const float (&x)[EPL], const SignMask& signs,
                                                  const Table16& thr, uint8_t* idx_s, uint32_t* prow,
                                                  float* norm_out, int lane) {
  constexpr int DIM = EPL * 32;
  constexpr int VPW = vals_per_word(BITS);
  constexpr int PDIM = packed_words(DIM, BITS);
  float sq[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) sq[j] = __fmul_rn(x[j], x[j]);
#pragma unroll
  for (int h = 1; h < EPL; h <<= 1) {
#pragma unroll
    for (int j = 0; j < EPL; j += 2 * h) sq[j] = __fadd_rn(sq[j], sq[j + h]);
  }
  float ss = sq[0];
#pragma unroll
  for (int k = 1; k < 32; k <<= 1) ss = __fadd_rn(ss, __shfl_xor_sync(0xffffffffu, ss, k));
  const float nrm = __fsqrt_rn(ss);
  const float safe = fmaxf(nrm, 1e-8f);

  float t[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    const float u = __fdiv_rn(x[j], safe);
    t[j] = __uint_as_float(__float_as_uint(u) ^ sign_bit_at(signs, lane * EPL + j));   // u * (+/-1), exact
  }
  warp_butterfly<EPL>(t, lane);

#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    int idx = 0;
#pragma unroll
    for (int b = 0; b < (1 << BITS) - 1; ++b) idx += (t[j] > thr.v[b]) ? 1 : 0;
    idx_s[lane * EPL + j] = (uint8_t)idx;
  }
  __syncwarp();
  for (int w = lane; w < PDIM; w += 32) {
    uint32_t word = 0;
#pragma unroll
    for (int k = 0; k < VPW; ++k) {
      const int e = w * VPW + k;
      if (e < DIM) word |= (uint32_t)idx_s[e] << (k * BITS);
    }
    prow[w] = word;
  }
  if (lane == 0) *norm_out = nrm;
  __syncwarp();
}

}  // namespace tq
