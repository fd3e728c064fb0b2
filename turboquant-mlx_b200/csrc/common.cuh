// Shared host/device helpers for libtqb200 (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tqb200.h"

namespace tq {

// ---- host-side error plumbing ------------------------------------------------
int set_error(int code, const char* fmt, ...);
int check_launch(const char* what);

#define TQ_REQUIRE(cond, code, ...)                         \
  do {                                                      \
    if (!(cond)) return ::tq::set_error((code), __VA_ARGS__); \
  } while (0)

// ---- codebook-sized parameters passed by value ---------------------------------
struct SignMask {       // bit e set  <=>  signs[e] == -1
  uint32_t w[8];
};
struct Table16 {        // centroids, or compare thresholds (unused tail = +inf)
  float v[16];
};

int make_sign_mask(const float* signs_host, int dim, SignMask* out);  // validates +/-1
int check_dim_bits(int dim, int bits, int max_dim);
// Thresholds T_i on the RAW butterfly output such that
//   ((raw * s) / s > boundary_i)  <=>  (raw > T_i),   s = float32(1/sqrt(dim)).
// The map raw -> (raw * s) / s is monotone, so T_i is the largest float whose
// image does not exceed the boundary; it is found by stepping ulps around it.
void make_raw_thresholds(const float* boundaries_host, int n, int dim, Table16* out);
int num_sms();

__host__ __device__ constexpr int vals_per_word(int bits) {
  return bits == 1 ? 32 : bits == 2 ? 16 : bits == 3 ? 10 : 8;
}
__host__ __device__ constexpr int packed_words(int dim, int bits) {
  return (dim + vals_per_word(bits) - 1) / vals_per_word(bits);
}

#ifdef __CUDACC__
// ---- device helpers ----------------------------------------------------------------
__device__ __forceinline__ float sign_at(const SignMask& m, int e) {
  return ((m.w[e >> 5] >> (e & 31)) & 1u) ? -1.0f : 1.0f;
}
__device__ __forceinline__ uint32_t sign_bit_at(const SignMask& m, int e) {
  return ((m.w[e >> 5] >> (e & 31)) & 1u) << 31;
}

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

// Raw Walsh-Hadamard butterfly of a vector spread over one warp: lane l holds
// elements [EPL*l, EPL*l + EPL).  Stage h pairs (j, j+h) -> (a+b, a-b) exactly
// as the reference's butterfly does, so results are bit-identical to a
// sequential float32 implementation.
template <int EPL>
__device__ __forceinline__ void warp_butterfly(float (&v)[EPL], int lane) {
#pragma unroll
  for (int h = 1; h < EPL; h <<= 1) {
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      if ((j & h) == 0) {
        float a = v[j], b = v[j + h];
        v[j] = __fadd_rn(a, b);
        v[j + h] = __fsub_rn(a, b);
      }
    }
  }
#pragma unroll
  for (int k = 1; k < 32; k <<= 1) {
    // upper partner: o - v = fma(v, -1, o), which rounds exactly like the subtraction it replaces
    const float sg = (lane & k) ? -1.0f : 1.0f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) v[j] = __fmaf_rn(v[j], sg, __shfl_xor_sync(0xffffffffu, v[j], k));
  }
}

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) x += __shfl_xor_sync(0xffffffffu, x, k);
  return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int k = 16; k > 0; k >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, k));
  return x;
}
#endif  // __CUDACC__

}  // namespace tq
