// PolarQuant encode / decode kernels and the Hadamard rotation helpers.
//
// Generic layout: one warp per vector, lane l holds elements [EPL*l, EPL*l+EPL)
// with EPL = dim / 32, so the butterfly runs log2(EPL) stages in registers and
// five stages through warp shuffles.  All float32 steps that feed the index
// compare use explicit round-to-nearest intrinsics (no FMA contraction) so the
// packed words are bit-identical to a sequential float32 evaluation.
#include "common.cuh"
#include "quantize_row.cuh"

namespace tq {

int try_launch_quantize_fast(const void* x, int x_dtype, int64_t n_outer, int64_t n_inner,
                             int64_t x_outer_stride, int dim, int bits, const SignMask& signs,
                             const Table16& thr, uint32_t* packed, int64_t packed_outer_stride,
                             float* norms, int64_t norms_outer_stride, cudaStream_t st);

int try_launch_dequantize_fast(const uint32_t* packed, int64_t packed_outer_stride, const float* norms,
                               int64_t norms_outer_stride, int64_t n_outer, int64_t n_inner, int dim,
                               int bits, const Table16& cs, float s, const SignMask& signs, void* out,
                               int out_dtype, int64_t out_outer_stride, cudaStream_t st);

constexpr int kWarpsPerBlock = 8;

struct QuantArgs {
  const void* x;
  int64_t n_vecs, n_inner, x_outer_stride;
  uint32_t* packed;
  int64_t packed_outer_stride;
  float* norms;
  int64_t norms_outer_stride;
  SignMask signs;
  Table16 thr;   // thresholds on the raw butterfly output
  int n_thr;
  // optional row copy done by extra blocks of the same launch (the dense K rows of a cache append)
  int q_blocks;              // blocks that quantize; blocks beyond copy (0: no copy job)
  const uint4* cp_src;
  uint4* cp_dst;
  int64_t cp_rows, cp_row16, cp_src_stride16, cp_dst_stride16;   // 16-byte units
};

template <typename T, int EPL, int BITS>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
quantize_warp_kernel(const QuantArgs a) {
  constexpr int DIM = EPL * 32;
  constexpr int PDIM = packed_words(DIM, BITS);
  __shared__ uint8_t idx_s[kWarpsPerBlock][DIM];
  // A kernel launched behind this one with programmatic stream serialization (the decode
  // attention after a cache append) may be scheduled now; it waits for this grid's completion
  // before it reads anything written here.
  if (threadIdx.x == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int q_blocks = a.q_blocks > 0 ? a.q_blocks : (int)gridDim.x;
  if ((int)blockIdx.x >= q_blocks) {      // copy blocks: rows of 16-byte chunks, strided on both sides
    const int64_t total = a.cp_rows * a.cp_row16;
    const int64_t step = (int64_t)(gridDim.x - q_blocks) * blockDim.x;
    for (int64_t i = (int64_t)(blockIdx.x - q_blocks) * blockDim.x + threadIdx.x; i < total; i += step) {
      const int64_t r = i / a.cp_row16, c = i - r * a.cp_row16;
      a.cp_dst[r * a.cp_dst_stride16 + c] = a.cp_src[r * a.cp_src_stride16 + c];
    }
    return;
  }
  const int64_t warp_global = (int64_t)blockIdx.x * kWarpsPerBlock + warp;
  const int64_t warp_stride = (int64_t)q_blocks * kWarpsPerBlock;

  for (int64_t v = warp_global; v < a.n_vecs; v += warp_stride) {
    const int64_t o = v / a.n_inner, i = v - o * a.n_inner;
    const T* row = reinterpret_cast<const T*>(a.x) + o * a.x_outer_stride + i * DIM + lane * EPL;
    float x[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) x[j] = to_f32<T>(row[j]);
    quantize_row_warp<EPL, BITS>(x, a.signs, a.thr, idx_s[warp], a.packed + o * a.packed_outer_stride + i * PDIM,
                                 a.norms + o * a.norms_outer_stride + i, lane);
  }
}

struct DequantArgs {
  const uint32_t* packed;
  int64_t packed_outer_stride;
  const float* norms;
  int64_t norms_outer_stride;
  int64_t n_vecs, n_inner;
  void* out;
  int64_t out_outer_stride;
  SignMask signs;
  Table16 cs;    // centroid * s
  float s;
};

template <typename T, int EPL, int BITS>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
dequantize_warp_kernel(const DequantArgs a) {
  constexpr int DIM = EPL * 32;
  constexpr int VPW = vals_per_word(BITS);
  constexpr int PDIM = packed_words(DIM, BITS);
  __shared__ float cs_s[16];
  if (threadIdx.x < 16) cs_s[threadIdx.x] = a.cs.v[threadIdx.x];
  __syncthreads();

  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int64_t warp_global = (int64_t)blockIdx.x * kWarpsPerBlock + warp;
  const int64_t warp_stride = (int64_t)gridDim.x * kWarpsPerBlock;

  float sgn[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) sgn[j] = sign_at(a.signs, lane * EPL + j);

  for (int64_t v = warp_global; v < a.n_vecs; v += warp_stride) {
    const int64_t o = v / a.n_inner, i = v - o * a.n_inner;
    const uint32_t* prow = a.packed + o * a.packed_outer_stride + i * PDIM;
    const float nrm = a.norms[o * a.norms_outer_stride + i];
    float y[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int e = lane * EPL + j;
      const uint32_t word = __ldg(prow + e / VPW);
      y[j] = cs_s[(word >> ((e % VPW) * BITS)) & ((1u << BITS) - 1u)];
    }
    warp_butterfly<EPL>(y, lane);
    T* orow = reinterpret_cast<T*>(a.out) + o * a.out_outer_stride + i * DIM + lane * EPL;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      // ((bfly * s) * signs) * norm, left to right as the reference writes it
      float r = __fmul_rn(__fmul_rn(__fmul_rn(y[j], a.s), sgn[j]), nrm);
      orow[j] = from_f32<T>(r);
    }
  }
}

struct HadamardArgs {
  const void* x;
  int64_t n_rows, in_row_stride;
  float* out;
  SignMask pre, post;
  int use_pre, use_post, normalize;
  float s;
};

template <typename T, int EPL>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
hadamard_warp_kernel(const HadamardArgs a) {
  constexpr int DIM = EPL * 32;
  const int lane = threadIdx.x & 31;
  const int warp = threadIdx.x >> 5;
  const int64_t warp_global = (int64_t)blockIdx.x * kWarpsPerBlock + warp;
  const int64_t warp_stride = (int64_t)gridDim.x * kWarpsPerBlock;
  for (int64_t v = warp_global; v < a.n_rows; v += warp_stride) {
    const T* row = reinterpret_cast<const T*>(a.x) + v * a.in_row_stride + lane * EPL;
    float t[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      float x = to_f32<T>(row[j]);
      t[j] = a.use_pre ? __fmul_rn(x, sign_at(a.pre, lane * EPL + j)) : x;
    }
    warp_butterfly<EPL>(t, lane);
    float* orow = a.out + v * DIM + lane * EPL;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      float r = a.normalize ? __fmul_rn(t[j], a.s) : t[j];
      if (a.use_post) r = __fmul_rn(r, sign_at(a.post, lane * EPL + j));
      orow[j] = r;
    }
  }
}

static int grid_for(int64_t n_vecs) {
  int64_t blocks = (n_vecs + kWarpsPerBlock - 1) / kWarpsPerBlock;
  int64_t cap = (int64_t)num_sms() * 8;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

template <typename T, int EPL>
static int launch_quantize_bits(const QuantArgs& a_in, int bits, cudaStream_t st) {
  QuantArgs a = a_in;
  int grid = grid_for(a.n_vecs);
  const int block = kWarpsPerBlock * 32;
  if (a.cp_rows > 0) {       // add copy blocks: 256 chunks of 16 bytes per block, at most 64 blocks
    a.q_blocks = grid;
    const int64_t chunks = a.cp_rows * a.cp_row16;
    int64_t cb = (chunks + block - 1) / block;
    grid += (int)(cb > 64 ? 64 : cb);
  }
  switch (bits) {
    case 1: quantize_warp_kernel<T, EPL, 1><<<grid, block, 0, st>>>(a); break;
    case 2: quantize_warp_kernel<T, EPL, 2><<<grid, block, 0, st>>>(a); break;
    case 3: quantize_warp_kernel<T, EPL, 3><<<grid, block, 0, st>>>(a); break;
    default: quantize_warp_kernel<T, EPL, 4><<<grid, block, 0, st>>>(a); break;
  }
  return check_launch("tq_quantize");
}
template <typename T>
static int launch_quantize(const QuantArgs& a, int dim, int bits, cudaStream_t st) {
  switch (dim) {
    case 32: return launch_quantize_bits<T, 1>(a, bits, st);
    case 64: return launch_quantize_bits<T, 2>(a, bits, st);
    case 128: return launch_quantize_bits<T, 4>(a, bits, st);
    default: return launch_quantize_bits<T, 8>(a, bits, st);
  }
}

template <typename T, int EPL>
static int launch_dequantize_bits(const DequantArgs& a, int bits, cudaStream_t st) {
  const int grid = grid_for(a.n_vecs);
  const int block = kWarpsPerBlock * 32;
  switch (bits) {
    case 1: dequantize_warp_kernel<T, EPL, 1><<<grid, block, 0, st>>>(a); break;
    case 2: dequantize_warp_kernel<T, EPL, 2><<<grid, block, 0, st>>>(a); break;
    case 3: dequantize_warp_kernel<T, EPL, 3><<<grid, block, 0, st>>>(a); break;
    default: dequantize_warp_kernel<T, EPL, 4><<<grid, block, 0, st>>>(a); break;
  }
  return check_launch("tq_dequantize");
}
template <typename T>
static int launch_dequantize(const DequantArgs& a, int dim, int bits, cudaStream_t st) {
  switch (dim) {
    case 32: return launch_dequantize_bits<T, 1>(a, bits, st);
    case 64: return launch_dequantize_bits<T, 2>(a, bits, st);
    case 128: return launch_dequantize_bits<T, 4>(a, bits, st);
    default: return launch_dequantize_bits<T, 8>(a, bits, st);
  }
}

template <typename T>
static int launch_hadamard(const HadamardArgs& a, int dim, cudaStream_t st) {
  const int grid = grid_for(a.n_rows);
  const int block = kWarpsPerBlock * 32;
  switch (dim) {
    case 32: hadamard_warp_kernel<T, 1><<<grid, block, 0, st>>>(a); break;
    case 64: hadamard_warp_kernel<T, 2><<<grid, block, 0, st>>>(a); break;
    case 128: hadamard_warp_kernel<T, 4><<<grid, block, 0, st>>>(a); break;
    default: hadamard_warp_kernel<T, 8><<<grid, block, 0, st>>>(a); break;
  }
  return check_launch("tq_hadamard");
}

}  // namespace tq

using namespace tq;

namespace {
struct RowCopy {
  const void* src;
  void* dst;
  int64_t rows, row_bytes, src_stride_bytes, dst_stride_bytes;
};
}  // namespace

static int quantize_impl(const void* x, int x_dtype, int64_t n_outer, int64_t n_inner,
                         int64_t x_outer_stride, int dim, int bits, const float* signs_host,
                         const float* boundaries_host, uint32_t* packed,
                         int64_t packed_outer_stride, float* norms, int64_t norms_outer_stride,
                         const RowCopy* copy, void* stream) {
  int rc = check_dim_bits(dim, bits, 256);
  if (rc) return rc;
  TQ_REQUIRE(n_outer >= 0 && n_inner >= 0, TQ_ERR_BAD_ARG, "negative vector count");
  TQ_REQUIRE(boundaries_host != nullptr, TQ_ERR_BAD_ARG, "boundaries pointer is NULL");
  if (n_outer * n_inner == 0) return TQ_OK;
  TQ_REQUIRE(x && packed && norms, TQ_ERR_BAD_ARG, "NULL tensor pointer");
  QuantArgs a;
  a.q_blocks = 0;
  a.cp_src = nullptr;
  a.cp_dst = nullptr;
  a.cp_rows = a.cp_row16 = a.cp_src_stride16 = a.cp_dst_stride16 = 0;
  if (copy) {
    a.cp_src = static_cast<const uint4*>(copy->src);
    a.cp_dst = static_cast<uint4*>(copy->dst);
    a.cp_rows = copy->rows;
    a.cp_row16 = copy->row_bytes / 16;
    a.cp_src_stride16 = copy->src_stride_bytes / 16;
    a.cp_dst_stride16 = copy->dst_stride_bytes / 16;
  }
  a.x = x;
  a.n_vecs = n_outer * n_inner;
  a.n_inner = n_inner;
  a.x_outer_stride = x_outer_stride;
  a.packed = packed;
  a.packed_outer_stride = packed_outer_stride;
  a.norms = norms;
  a.norms_outer_stride = norms_outer_stride;
  rc = make_sign_mask(signs_host, dim, &a.signs);
  if (rc) return rc;
  a.n_thr = (1 << bits) - 1;
  make_raw_thresholds(boundaries_host, a.n_thr, dim, &a.thr);
  cudaStream_t st = (cudaStream_t)stream;
  if (x_dtype < TQ_F32 || x_dtype > TQ_BF16) return set_error(TQ_ERR_BAD_ARG, "unknown dtype %d", x_dtype);
  if (!copy) {   // large contiguous dim-128 batches: split-per-vector kernel
    rc = try_launch_quantize_fast(x, x_dtype, n_outer, n_inner, x_outer_stride, dim, bits, a.signs, a.thr,
                                  packed, packed_outer_stride, norms, norms_outer_stride, st);
    if (rc != TQ_ERR_UNSUPPORTED) return rc;
  }
  switch (x_dtype) {
    case TQ_F32: return launch_quantize<float>(a, dim, bits, st);
    case TQ_F16: return launch_quantize<__half>(a, dim, bits, st);
    case TQ_BF16: return launch_quantize<__nv_bfloat16>(a, dim, bits, st);
    default: return set_error(TQ_ERR_BAD_ARG, "unknown dtype %d", x_dtype);
  }
}

extern "C" int tq_quantize(const void* x, int x_dtype, int64_t n_outer, int64_t n_inner,
                           int64_t x_outer_stride, int dim, int bits, const float* signs_host,
                           const float* boundaries_host, uint32_t* packed,
                           int64_t packed_outer_stride, float* norms, int64_t norms_outer_stride,
                           void* stream) {
  return quantize_impl(x, x_dtype, n_outer, n_inner, x_outer_stride, dim, bits, signs_host, boundaries_host,
                       packed, packed_outer_stride, norms, norms_outer_stride, nullptr, stream);
}

extern "C" int tq_quantize_append(const void* x, int x_dtype, int64_t n_outer, int64_t n_inner,
                                  int64_t x_outer_stride, int dim, int bits, const float* signs_host,
                                  const float* boundaries_host, uint32_t* packed,
                                  int64_t packed_outer_stride, float* norms, int64_t norms_outer_stride,
                                  const void* copy_src, void* copy_dst, int64_t copy_rows,
                                  int64_t copy_row_bytes, int64_t copy_src_stride_bytes,
                                  int64_t copy_dst_stride_bytes, void* stream) {
  TQ_REQUIRE(n_outer * n_inner > 0, TQ_ERR_BAD_ARG, "tq_quantize_append needs at least one vector");
  TQ_REQUIRE(copy_src && copy_dst && copy_rows > 0 && copy_row_bytes > 0, TQ_ERR_BAD_ARG, "empty copy job");
  TQ_REQUIRE(((reinterpret_cast<uintptr_t>(copy_src) | reinterpret_cast<uintptr_t>(copy_dst) |
               (uintptr_t)copy_row_bytes | (uintptr_t)copy_src_stride_bytes | (uintptr_t)copy_dst_stride_bytes) & 15) == 0,
             TQ_ERR_MISALIGNED, "copy rows must be 16-byte multiples at 16-byte boundaries");
  const RowCopy rc = {copy_src, copy_dst, copy_rows, copy_row_bytes, copy_src_stride_bytes, copy_dst_stride_bytes};
  return quantize_impl(x, x_dtype, n_outer, n_inner, x_outer_stride, dim, bits, signs_host, boundaries_host,
                       packed, packed_outer_stride, norms, norms_outer_stride, &rc, stream);
}

extern "C" int tq_dequantize(const uint32_t* packed, int64_t packed_outer_stride,
                             const float* norms, int64_t norms_outer_stride, int64_t n_outer,
                             int64_t n_inner, int dim, int bits, const float* centroids_host,
                             const float* signs_host, void* out, int out_dtype,
                             int64_t out_outer_stride, void* stream) {
  int rc = check_dim_bits(dim, bits, 256);
  if (rc) return rc;
  TQ_REQUIRE(n_outer >= 0 && n_inner >= 0, TQ_ERR_BAD_ARG, "negative vector count");
  TQ_REQUIRE(centroids_host != nullptr, TQ_ERR_BAD_ARG, "centroids pointer is NULL");
  if (n_outer * n_inner == 0) return TQ_OK;
  TQ_REQUIRE(packed && norms && out, TQ_ERR_BAD_ARG, "NULL tensor pointer");
  DequantArgs a;
  a.packed = packed;
  a.packed_outer_stride = packed_outer_stride;
  a.norms = norms;
  a.norms_outer_stride = norms_outer_stride;
  a.n_vecs = n_outer * n_inner;
  a.n_inner = n_inner;
  a.out = out;
  a.out_outer_stride = out_outer_stride;
  rc = make_sign_mask(signs_host, dim, &a.signs);
  if (rc) return rc;
  a.s = (float)(1.0 / sqrt((double)dim));
  for (int i = 0; i < 16; ++i) {
    volatile float cs = (i < (1 << bits)) ? centroids_host[i] * a.s : 0.0f;
    a.cs.v[i] = cs;
  }
  cudaStream_t st = (cudaStream_t)stream;
  {   // large contiguous dim-128 batches: split-per-vector kernel
    rc = try_launch_dequantize_fast(packed, packed_outer_stride, norms, norms_outer_stride, n_outer, n_inner,
                                    dim, bits, a.cs, a.s, a.signs, out, out_dtype, out_outer_stride, st);
    if (rc != TQ_ERR_UNSUPPORTED) return rc;
  }
  switch (out_dtype) {
    case TQ_F32: return launch_dequantize<float>(a, dim, bits, st);
    case TQ_F16: return launch_dequantize<__half>(a, dim, bits, st);
    case TQ_BF16: return launch_dequantize<__nv_bfloat16>(a, dim, bits, st);
    default: return set_error(TQ_ERR_BAD_ARG, "unknown dtype %d", out_dtype);
  }
}

static int hadamard_common(const void* x, int dtype, int64_t n_rows, int64_t in_stride, int dim,
                           const float* pre, const float* post, int normalize, float* out,
                           void* stream, const char* who) {
  int rc = check_dim_bits(dim, 3, 256);
  if (rc) return rc;
  if (n_rows <= 0) return TQ_OK;
  TQ_REQUIRE(x && out, TQ_ERR_BAD_ARG, "%s: NULL tensor pointer", who);
  HadamardArgs a;
  a.x = x;
  a.n_rows = n_rows;
  a.in_row_stride = in_stride;
  a.out = out;
  a.use_pre = pre != nullptr;
  a.use_post = post != nullptr;
  a.normalize = normalize;
  a.s = (float)(1.0 / sqrt((double)dim));
  if (pre && (rc = make_sign_mask(pre, dim, &a.pre))) return rc;
  if (post && (rc = make_sign_mask(post, dim, &a.post))) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dtype) {
    case TQ_F32: return launch_hadamard<float>(a, dim, st);
    case TQ_F16: return launch_hadamard<__half>(a, dim, st);
    case TQ_BF16: return launch_hadamard<__nv_bfloat16>(a, dim, st);
    default: return set_error(TQ_ERR_BAD_ARG, "unknown dtype %d", dtype);
  }
}

extern "C" int tq_prerotate_query(const void* q, int q_dtype, int64_t n_heads,
                                  int64_t q_head_stride, int dim, const float* signs_host,
                                  float* out, void* stream) {
  TQ_REQUIRE(signs_host != nullptr, TQ_ERR_BAD_ARG, "signs pointer is NULL");
  return hadamard_common(q, q_dtype, n_heads, q_head_stride, dim, signs_host, nullptr, 0, out,
                         stream, "tq_prerotate_query");
}

extern "C" int tq_hadamard(const float* x, int64_t n_rows, int dim, const float* pre_signs_host,
                           const float* post_signs_host, int normalize, float* out,
                           void* stream) {
  return hadamard_common(x, TQ_F32, n_rows, dim, dim, pre_signs_host, post_signs_host, normalize,
                         out, stream, "tq_hadamard");
}
