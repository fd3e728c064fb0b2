// Group-wise affine quantisation (K8 / V4): one warp per group of `group`
// consecutive elements.  scale = fp16((max - min) / (2^bits - 1)), bias =
// fp16(min), code = clip(rint((x - bias) / scale), 0, 2^bits - 1).
#include "common.cuh"

namespace tq {

template <typename T, int EPG>
__global__ void __launch_bounds__(256)
affine_quantize_kernel(const T* __restrict__ x, int64_t n_groups, int bits,
                       uint8_t* __restrict__ codes, __half* __restrict__ scales,
                       __half* __restrict__ biases, int gpr /* groups per row */, int64_t x_row_stride,
                       int64_t codes_row_stride /* bytes */, int64_t sb_row_stride,
                       const int* __restrict__ pos_dev, int64_t codes_pos_stride, int64_t sb_pos_stride) {
  constexpr int GROUP = EPG * 32;
  if (pos_dev != nullptr) {   // destination rows start at a position that lives on the device
    const int64_t pos = *pos_dev;
    codes += pos * codes_pos_stride;
    scales += pos * sb_pos_stride;
    biases += pos * sb_pos_stride;
  }
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int64_t warp_stride = (int64_t)gridDim.x * 8;
  const float qmax = (float)((1 << bits) - 1);
  for (int64_t g = warp_global; g < n_groups; g += warp_stride) {
    const int64_t row = g / gpr;
    const int gi = (int)(g - row * gpr);
    const T* src = x + row * x_row_stride + gi * GROUP + lane * EPG;
    float v[EPG];
    float lo = INFINITY, hi = -INFINITY;
#pragma unroll
    for (int j = 0; j < EPG; ++j) {
      v[j] = to_f32<T>(src[j]);
      lo = fminf(lo, v[j]);
      hi = fmaxf(hi, v[j]);
    }
#pragma unroll
    for (int k = 16; k > 0; k >>= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, k));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, k));
    }
    const __half sc_h = __float2half_rn(__fdiv_rn(__fsub_rn(hi, lo), qmax));
    const __half bi_h = __float2half_rn(lo);
    const float sc = __half2float(sc_h), bi = __half2float(bi_h);
    int code[EPG];
#pragma unroll
    for (int j = 0; j < EPG; ++j) {
      float c = sc > 0.f ? rintf(__fdiv_rn(__fsub_rn(v[j], bi), sc)) : 0.f;
      code[j] = (int)fminf(fmaxf(c, 0.f), qmax);
    }
    if (bits == 8) {
      uint8_t* dst = codes + row * codes_row_stride + gi * GROUP + lane * EPG;
#pragma unroll
      for (int j = 0; j < EPG; ++j) dst[j] = (uint8_t)code[j];
    } else {  // 4-bit: two codes per byte, low nibble first
      uint8_t* dst = codes + row * codes_row_stride + (gi * GROUP + lane * EPG) / 2;
      if (EPG == 1) {
        const int other = __shfl_xor_sync(0xffffffffu, code[0], 1);
        if ((lane & 1) == 0) dst[0] = (uint8_t)(code[0] | (other << 4));
      } else {
#pragma unroll
        for (int j = 0; j < EPG; j += 2) dst[j / 2] = (uint8_t)(code[j] | (code[j + 1 < EPG ? j + 1 : j] << 4));
      }
    }
    if (lane == 0) {
      scales[row * sb_row_stride + gi] = sc_h;
      biases[row * sb_row_stride + gi] = bi_h;
    }
  }
}

template <typename T>
__global__ void affine_dequantize_kernel(const uint8_t* __restrict__ codes,
                                         const __half* __restrict__ scales,
                                         const __half* __restrict__ biases, int64_t n_elems,
                                         int group, int bits, T* __restrict__ out) {
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_elems; i += stride) {
    const int code = bits == 8 ? codes[i] : ((codes[i >> 1] >> ((i & 1) * 4)) & 0xF);
    const int64_t g = i / group;
    out[i] = from_f32<T>(__half2float(scales[g]) * (float)code + __half2float(biases[g]));
  }
}

template <typename T>
static int launch_affine_q(const void* x, int64_t n_groups, int group, int bits, uint8_t* codes,
                           void* sc, void* bi, int gpr, int64_t xs, int64_t cs, int64_t ss, cudaStream_t st,
                           const int* pos = nullptr, int64_t cps = 0, int64_t sps = 0) {
  int64_t blocks = (n_groups + 7) / 8;
  const int64_t cap = (int64_t)num_sms() * 8;
  const int grid = (int)(blocks > cap ? cap : blocks);
  const T* xt = reinterpret_cast<const T*>(x);
  switch (group) {
    case 32: affine_quantize_kernel<T, 1><<<grid, 256, 0, st>>>(xt, n_groups, bits, codes, (__half*)sc, (__half*)bi, gpr, xs, cs, ss, pos, cps, sps); break;
    case 64: affine_quantize_kernel<T, 2><<<grid, 256, 0, st>>>(xt, n_groups, bits, codes, (__half*)sc, (__half*)bi, gpr, xs, cs, ss, pos, cps, sps); break;
    default: affine_quantize_kernel<T, 4><<<grid, 256, 0, st>>>(xt, n_groups, bits, codes, (__half*)sc, (__half*)bi, gpr, xs, cs, ss, pos, cps, sps); break;
  }
  return check_launch("tq_affine_quantize");
}

}  // namespace tq

using namespace tq;

static int affine_check(int dim, int group, int bits) {
  TQ_REQUIRE(group == 32 || group == 64 || group == 128, TQ_ERR_BAD_ARG,
             "group must be 32, 64 or 128, got %d", group);
  TQ_REQUIRE(dim > 0 && dim % group == 0, TQ_ERR_BAD_DIM, "dim %d is not a multiple of group %d", dim, group);
  TQ_REQUIRE(bits == 4 || bits == 8, TQ_ERR_BAD_BITS, "affine bits must be 4 or 8, got %d", bits);
  return TQ_OK;
}

extern "C" int tq_affine_quantize_rows(const void* x, int x_dtype, int64_t n_rows, int dim, int group,
                                       int bits, int64_t x_row_stride, uint8_t* codes, int64_t codes_row_stride,
                                       void* scales_f16, void* biases_f16, int64_t sb_row_stride, void* stream) {
  return tq_affine_quantize_rows_at(x, x_dtype, n_rows, dim, group, bits, x_row_stride, codes, codes_row_stride,
                                    scales_f16, biases_f16, sb_row_stride, nullptr, 0, 0, stream);
}

extern "C" int tq_affine_quantize_rows_at(const void* x, int x_dtype, int64_t n_rows, int dim, int group,
                                          int bits, int64_t x_row_stride, uint8_t* codes, int64_t codes_row_stride,
                                          void* scales_f16, void* biases_f16, int64_t sb_row_stride,
                                          const int32_t* position_dev, int64_t codes_pos_stride,
                                          int64_t sb_pos_stride, void* stream) {
  int rc = affine_check(dim, group, bits);
  if (rc) return rc;
  if (n_rows <= 0) return TQ_OK;
  TQ_REQUIRE(x && codes && scales_f16 && biases_f16, TQ_ERR_BAD_ARG, "NULL tensor pointer");
  const int gpr = dim / group;
  TQ_REQUIRE(x_row_stride >= dim && codes_row_stride >= (bits == 8 ? dim : dim / 2) && sb_row_stride >= gpr,
             TQ_ERR_BAD_ARG, "row strides shorter than a row");
  const int64_t n_groups = n_rows * gpr;
  cudaStream_t st = (cudaStream_t)stream;
  switch (x_dtype) {
    case TQ_F32:
      return launch_affine_q<float>(x, n_groups, group, bits, codes, scales_f16, biases_f16, gpr, x_row_stride,
                                    codes_row_stride, sb_row_stride, st, position_dev, codes_pos_stride, sb_pos_stride);
    case TQ_F16:
      return launch_affine_q<__half>(x, n_groups, group, bits, codes, scales_f16, biases_f16, gpr, x_row_stride,
                                     codes_row_stride, sb_row_stride, st, position_dev, codes_pos_stride, sb_pos_stride);
    case TQ_BF16:
      return launch_affine_q<__nv_bfloat16>(x, n_groups, group, bits, codes, scales_f16, biases_f16, gpr,
                                            x_row_stride, codes_row_stride, sb_row_stride, st, position_dev,
                                            codes_pos_stride, sb_pos_stride);
    default: return set_error(TQ_ERR_BAD_ARG, "unknown dtype %d", x_dtype);
  }
}

extern "C" int tq_affine_quantize(const void* x, int x_dtype, int64_t n_rows, int dim, int group,
                                  int bits, uint8_t* codes, void* scales_f16, void* biases_f16,
                                  void* stream) {
  int rc = affine_check(dim, group, bits);
  if (rc) return rc;
  return tq_affine_quantize_rows(x, x_dtype, n_rows, dim, group, bits, dim, codes, bits == 8 ? dim : dim / 2,
                                 scales_f16, biases_f16, dim / group, stream);
}

extern "C" int tq_affine_dequantize(const uint8_t* codes, const void* scales_f16,
                                    const void* biases_f16, int64_t n_rows, int dim, int group,
                                    int bits, void* out, int out_dtype, void* stream) {
  int rc = affine_check(dim, group, bits);
  if (rc) return rc;
  if (n_rows <= 0) return TQ_OK;
  TQ_REQUIRE(codes && scales_f16 && biases_f16 && out, TQ_ERR_BAD_ARG, "NULL tensor pointer");
  const int64_t n = n_rows * dim;
  int64_t blocks = (n + 255) / 256;
  const int64_t cap = (int64_t)num_sms() * 16;
  const int grid = (int)(blocks > cap ? cap : blocks);
  cudaStream_t st = (cudaStream_t)stream;
  const __half* sc = (const __half*)scales_f16;
  const __half* bi = (const __half*)biases_f16;
  switch (out_dtype) {
    case TQ_F32: affine_dequantize_kernel<float><<<grid, 256, 0, st>>>(codes, sc, bi, n, group, bits, (float*)out); break;
    case TQ_F16: affine_dequantize_kernel<__half><<<grid, 256, 0, st>>>(codes, sc, bi, n, group, bits, (__half*)out); break;
    case TQ_BF16: affine_dequantize_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(codes, sc, bi, n, group, bits, (__nv_bfloat16*)out); break;
    default: return set_error(TQ_ERR_BAD_ARG, "unknown dtype %d", out_dtype);
  }
  return check_launch("tq_affine_dequantize");
}
