// Attention-side kernels, float32 CUDA-core versions that accept every supported
// shape (dim 32..256, bits 1..4, any n_rep, polar / dense / affine keys, polar /
// affine values, additive mask).  The tensor-core specialisation for dim 128
// lives in flash_mma.cu; this file is the general path and owns the split-K
// merge that both share.
#include <math.h>

#include "common.cuh"
#include "flash.cuh"

namespace tq {

// ---------------------------------------------------------------------------
// Q.K scores with a pre-rotated query (metal_kernels_v4.py:71-113)
// ---------------------------------------------------------------------------
constexpr int kScoreWarps = 8;
constexpr int kScorePosPerBlock = 64;

template <int EPL, int BITS>
__global__ void __launch_bounds__(kScoreWarps * 32)
prerot_scores_kernel(const float* __restrict__ q_rot, const uint32_t* __restrict__ k_packed,
                     int64_t k_head_stride, const float* __restrict__ k_norms,
                     int64_t kn_head_stride, int64_t seq, int n_rep, Table16 cent, float inv_dim,
                     float* __restrict__ out) {
  constexpr int DIM = EPL * 32;
  constexpr int VPW = vals_per_word(BITS);
  constexpr int PDIM = packed_words(DIM, BITS);
  extern __shared__ float q_s[];  // n_rep * DIM
  __shared__ float cent_s[16];
  const int kvh = blockIdx.y;
  for (int i = threadIdx.x; i < n_rep * DIM; i += blockDim.x)
    q_s[i] = q_rot[(int64_t)kvh * n_rep * DIM + i];
  if (threadIdx.x < 16) cent_s[threadIdx.x] = cent.v[threadIdx.x];
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t p0 = (int64_t)blockIdx.x * kScorePosPerBlock;
  for (int pi = warp; pi < kScorePosPerBlock; pi += kScoreWarps) {
    const int64_t p = p0 + pi;
    if (p >= seq) break;
    const uint32_t* row = k_packed + kvh * k_head_stride + p * PDIM;
    float c[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int e = lane * EPL + j;
      c[j] = cent_s[(__ldg(row + e / VPW) >> ((e % VPW) * BITS)) & ((1u << BITS) - 1u)];
    }
    const float nrm = k_norms[kvh * kn_head_stride + p];
    for (int r = 0; r < n_rep; ++r) {
      float part = 0.f;
#pragma unroll
      for (int j = 0; j < EPL; ++j) part += c[j] * q_s[r * DIM + lane * EPL + j];
      part = warp_sum(part);
      if (lane == 0) out[((int64_t)kvh * n_rep + r) * seq + p] = part * nrm * inv_dim;
    }
  }
}

// Per-position dequant then dot with the raw query (kernels.py:58-117), MHA only.
template <int EPL, int BITS>
__global__ void __launch_bounds__(kScoreWarps * 32)
packed_scores_kernel(const float* __restrict__ query, const uint32_t* __restrict__ k_packed,
                     int64_t k_head_stride, const float* __restrict__ k_norms,
                     int64_t kn_head_stride, int64_t seq, Table16 cs, SignMask signs, float s,
                     float* __restrict__ out) {
  constexpr int DIM = EPL * 32;
  constexpr int VPW = vals_per_word(BITS);
  constexpr int PDIM = packed_words(DIM, BITS);
  __shared__ float cs_s[16];
  if (threadIdx.x < 16) cs_s[threadIdx.x] = cs.v[threadIdx.x];
  __syncthreads();
  const int h = blockIdx.y;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float q[EPL], sg[EPL];
#pragma unroll
  for (int j = 0; j < EPL; ++j) {
    q[j] = query[(int64_t)h * DIM + lane * EPL + j];
    sg[j] = sign_at(signs, lane * EPL + j);
  }
  const int64_t p0 = (int64_t)blockIdx.x * kScorePosPerBlock;
  for (int pi = warp; pi < kScorePosPerBlock; pi += kScoreWarps) {
    const int64_t p = p0 + pi;
    if (p >= seq) break;
    const uint32_t* row = k_packed + h * k_head_stride + p * PDIM;
    float y[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int e = lane * EPL + j;
      y[j] = cs_s[(__ldg(row + e / VPW) >> ((e % VPW) * BITS)) & ((1u << BITS) - 1u)];
    }
    warp_butterfly<EPL>(y, lane);
    const float nrm = k_norms[h * kn_head_stride + p];
    float part = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) part += (((y[j] * s) * sg[j]) * nrm) * q[j];
    part = warp_sum(part);
    if (lane == 0) out[(int64_t)h * seq + p] = part;
  }
}

// ---------------------------------------------------------------------------
// sparse_v_matvec (sparse_v.py:32-88): phase 1 partial sums per sequence chunk
// ---------------------------------------------------------------------------
constexpr int kSvRMax = 8;

template <int BITS>
__global__ void __launch_bounds__(256)
sparse_v_partial_kernel(const float* __restrict__ weights, int64_t w_head_stride,
                        const uint32_t* __restrict__ v_packed, int64_t v_head_stride,
                        const float* __restrict__ v_norms, int64_t vn_head_stride, int64_t seq,
                        int64_t chunk, int dim, int n_rep, float thr, Table16 cent,
                        float* __restrict__ ws /* (splits, n_q, dim) */, int n_q) {
  constexpr int VPW = vals_per_word(BITS);
  const int pdim = (dim + VPW - 1) / VPW;
  __shared__ float cent_s[16];
  __shared__ float red_s[kSvRMax][256];
  if (threadIdx.x < 16) cent_s[threadIdx.x] = cent.v[threadIdx.x];
  __syncthreads();
  const int py_n = 256 / dim;
  const int e = threadIdx.x % dim, py = threadIdx.x / dim;
  const int kvh = blockIdx.y;
  const int r0 = blockIdx.z * kSvRMax;
  const int nr = min(kSvRMax, n_rep - r0);
  const int64_t pb = (int64_t)blockIdx.x * chunk;
  const int64_t pe = min(seq, pb + chunk);
  const int widx = e / VPW, shift = (e % VPW) * BITS;
  float acc[kSvRMax];
#pragma unroll
  for (int r = 0; r < kSvRMax; ++r) acc[r] = 0.f;
  const uint32_t* vbase = v_packed + kvh * v_head_stride;
  const float* nbase = v_norms + kvh * vn_head_stride;
  const float* wbase = weights + ((int64_t)kvh * n_rep + r0) * w_head_stride;
  for (int64_t p = pb + py; p < pe; p += py_n) {
    float w[kSvRMax];
    bool any = false;
#pragma unroll
    for (int r = 0; r < kSvRMax; ++r) {
      w[r] = (r < nr) ? wbase[r * w_head_stride + p] : 0.f;
      any |= (r < nr) && !(w[r] < thr);
    }
    if (!any) continue;   // every head skips this position: no packed load at all
    const float c = cent_s[(__ldg(vbase + p * pdim + widx) >> shift) & ((1u << BITS) - 1u)];
    const float nrm = nbase[p];
#pragma unroll
    for (int r = 0; r < kSvRMax; ++r)
      if (r < nr && !(w[r] < thr)) acc[r] += (w[r] * nrm) * c;
  }
#pragma unroll
  for (int r = 0; r < kSvRMax; ++r) red_s[r][threadIdx.x] = acc[r];
  __syncthreads();
  if (py == 0) {
    for (int r = 0; r < nr; ++r) {
      float s = 0.f;
      for (int y = 0; y < py_n; ++y) s += red_s[r][y * dim + e];
      ws[((int64_t)blockIdx.x * n_q + kvh * n_rep + r0 + r) * dim + e] = s;
    }
  }
}

// phase 2: sum the chunk partials, one butterfly, signs and 1/dim
__global__ void sparse_v_finish_kernel(const float* __restrict__ ws, int splits, int n_q, int dim,
                                       SignMask signs, float inv_dim, float* __restrict__ out) {
  __shared__ float sh[256];
  const int h = blockIdx.x, e = threadIdx.x;
  float s = 0.f;
  for (int i = 0; i < splits; ++i) s += ws[((int64_t)i * n_q + h) * dim + e];
  sh[e] = s;
  __syncthreads();
  for (int hh = 1; hh < dim; hh <<= 1) {
    if ((e & hh) == 0) {
      float a = sh[e], b = sh[e + hh];
      sh[e] = a + b;
      sh[e + hh] = a - b;
    }
    __syncthreads();
  }
  out[(int64_t)h * dim + e] = sh[e] * sign_at(signs, e) * inv_dim;
}

// ---------------------------------------------------------------------------
// generic split-K flash decode
// ---------------------------------------------------------------------------
constexpr int kFgThreads = 256;
constexpr int kFgWarps = 8;
constexpr int kFgTile = 32;
constexpr int kFgRMax = 8;

template <typename T>
__device__ __forceinline__ float dense_at(const void* base, int64_t idx) {
  return to_f32<T>(reinterpret_cast<const T*>(base)[idx]);
}

template <int EPL>
__global__ void __launch_bounds__(kFgThreads)
flash_generic_kernel(const FlashArgs a) {
  constexpr int DIM = EPL * 32;
  constexpr int PY = kFgThreads / DIM;
  __shared__ float q_s[kFgRMax][DIM];
  __shared__ float s_s[kFgRMax][kFgTile];
  __shared__ float vn_s[kFgTile];
  __shared__ float alpha_s[kFgRMax], m_s[kFgRMax], l_s[kFgRMax];
  __shared__ float kc_s[16], vc_s[16];
  __shared__ float red_s[PY > 1 ? (PY - 1) * kFgRMax * DIM : 1];

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x;
  const int rgroups = (a.n_rep + kFgRMax - 1) / kFgRMax;
  const int kvh = blockIdx.y / rgroups;
  const int r0 = (blockIdx.y % rgroups) * kFgRMax;
  const int nr = min(kFgRMax, a.n_rep - r0);
  const int b = blockIdx.z;
  const int h0 = kvh * a.n_rep + r0;   // first query head of this block

  if (tid < 16) {
    kc_s[tid] = a.k_cent.v[tid];
    vc_s[tid] = a.v_cent.v[tid];
  }
  // query rows: load (times k signs when the kernel rotates), butterfly per warp
  if (warp < kFgRMax) {
    const int r = warp;
    float t[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      float v = 0.f;
      if (r < nr) {
        const int64_t off = b * a.q_batch_stride + (int64_t)(h0 + r) * a.q_head_stride + lane * EPL + j;
        v = a.q_dtype == TQ_F32 ? dense_at<float>(a.q, off)
            : a.q_dtype == TQ_F16 ? dense_at<__half>(a.q, off)
                                  : dense_at<__nv_bfloat16>(a.q, off);
      }
      t[j] = v;
    }
    if (a.k_format == TQ_KV_POLAR && !a.q_prerotated) {
#pragma unroll
      for (int j = 0; j < EPL; ++j) t[j] *= sign_at(a.k_signs, lane * EPL + j);
      warp_butterfly<EPL>(t, lane);
    }
#pragma unroll
    for (int j = 0; j < EPL; ++j) q_s[r][lane * EPL + j] = t[j];
  }
  if (tid < kFgRMax) {
    m_s[tid] = -INFINITY;
    l_s[tid] = 0.f;
    alpha_s[tid] = 1.f;
  }
  __syncthreads();

  const int64_t pb = (int64_t)split * a.chunk;
  const int64_t pe = min(a.seq_len, pb + a.chunk);
  const int kvpw = vals_per_word(a.k_bits), kpd = packed_words(DIM, a.k_bits);
  const int vvpw = vals_per_word(a.v_bits), vpd = packed_words(DIM, a.v_bits);
  const uint32_t kmask = (1u << a.k_bits) - 1u, vmask = (1u << a.v_bits) - 1u;
  const float inv_dim = 1.0f / DIM;

  // phase C ownership
  const int e = tid % DIM, py = tid / DIM;
  float acc[kFgRMax];
#pragma unroll
  for (int r = 0; r < kFgRMax; ++r) acc[r] = 0.f;

  for (int64_t t0 = pb; t0 < pe; t0 += kFgTile) {
    // ---- phase A: scores of the tile -------------------------------------
    for (int pi = warp; pi < kFgTile; pi += kFgWarps) {
      const int64_t p = t0 + pi;
      if (p >= pe) {
        if (lane < kFgRMax) s_s[lane][pi] = -INFINITY;
        if (lane == 0) vn_s[pi] = 0.f;
        continue;
      }
      float c[EPL];
      float post = a.attn_scale;
      if (a.k_format == TQ_KV_POLAR) {
        const uint32_t* row = reinterpret_cast<const uint32_t*>(a.k_data) + b * a.k_batch_stride +
                              kvh * a.k_head_stride + p * kpd;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
          const int ee = lane * EPL + j;
          c[j] = kc_s[(__ldg(row + ee / kvpw) >> ((ee % kvpw) * a.k_bits)) & kmask];
        }
        post = a.k_norms[b * a.kn_batch_stride + kvh * a.kn_head_stride + p] * inv_dim * a.attn_scale;
      } else if (a.k_format == TQ_KV_DENSE) {
        const int64_t off = b * a.k_batch_stride + kvh * a.k_head_stride + p * DIM + lane * EPL;
#pragma unroll
        for (int j = 0; j < EPL; ++j)
          c[j] = a.k_dtype == TQ_F32 ? dense_at<float>(a.k_data, off + j)
                 : a.k_dtype == TQ_F16 ? dense_at<__half>(a.k_data, off + j)
                                       : dense_at<__nv_bfloat16>(a.k_data, off + j);
      } else {  // affine, 8-bit codes
        const uint8_t* row = reinterpret_cast<const uint8_t*>(a.k_data) + b * a.k_batch_stride +
                             kvh * a.k_head_stride + p * DIM;
        const int ng = DIM / a.k_group;
        const int64_t soff = b * a.ks_batch_stride + kvh * a.ks_head_stride + p * ng;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
          const int ee = lane * EPL + j;
          const int g = ee / a.k_group;
          const float sc = __half2float(reinterpret_cast<const __half*>(a.k_scales)[soff + g]);
          const float bi = __half2float(reinterpret_cast<const __half*>(a.k_biases)[soff + g]);
          c[j] = sc * (float)row[ee] + bi;
        }
      }
      for (int r = 0; r < nr; ++r) {
        float part = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) part += c[j] * q_s[r][lane * EPL + j];
        part = warp_sum(part);
        if (lane == 0) {
          float sc = part * post;
          if (a.mask) sc += a.mask[b * a.mask_batch_stride + (int64_t)(h0 + r) * a.mask_head_stride + p];
          s_s[r][pi] = sc;
        }
      }
      if (lane == 0)
        vn_s[pi] = (a.v_format == TQ_KV_POLAR)
                       ? a.v_norms[b * a.vn_batch_stride + kvh * a.vn_head_stride + p]
                       : 1.f;
    }
    __syncthreads();
    // ---- phase B: online softmax, one warp per query head -------------------
    if (warp < nr) {
      const int r = warp;
      const float sc = s_s[r][lane];
      const float m_old = m_s[r];
      const float m_new = fmaxf(m_old, warp_max(sc));
      float alpha = 1.f, pexp = 0.f;
      if (m_new > -INFINITY) {
        alpha = __expf(m_old - m_new);
        pexp = __expf(sc - m_new);
      }
      const float lsum = warp_sum(pexp);
      s_s[r][lane] = pexp;
      if (lane == 0) {
        alpha_s[r] = alpha;
        m_s[r] = m_new;
        l_s[r] = l_s[r] * alpha + lsum;
      }
    }
    __syncthreads();
    // ---- phase C: accumulate in the rotated domain -----------------------------
#pragma unroll
    for (int r = 0; r < kFgRMax; ++r) acc[r] *= alpha_s[r];
    for (int pi = py; pi < kFgTile; pi += PY) {
      const int64_t p = t0 + pi;
      if (p >= pe) break;
      float val;
      if (a.v_format == TQ_KV_POLAR) {
        const uint32_t* row = reinterpret_cast<const uint32_t*>(a.v_data) + b * a.v_batch_stride +
                              kvh * a.v_head_stride + p * vpd;
        val = vc_s[(__ldg(row + e / vvpw) >> ((e % vvpw) * a.v_bits)) & vmask];
      } else {  // affine, 4- or 8-bit codes
        const int ng = DIM / a.v_group;
        const int64_t soff = b * a.vs_batch_stride + kvh * a.vs_head_stride + p * ng + e / a.v_group;
        const float sc = __half2float(reinterpret_cast<const __half*>(a.v_scales)[soff]);
        const float bi = __half2float(reinterpret_cast<const __half*>(a.v_biases)[soff]);
        const int row_bytes = a.v_bits == 4 ? DIM / 2 : DIM;
        const uint8_t* row = reinterpret_cast<const uint8_t*>(a.v_data) + b * a.v_batch_stride +
                             kvh * a.v_head_stride + p * row_bytes;
        const int code = a.v_bits == 4 ? ((row[e >> 1] >> ((e & 1) * 4)) & 0xF) : row[e];
        val = sc * (float)code + bi;
      }
      const float vn = vn_s[pi];
#pragma unroll
      for (int r = 0; r < kFgRMax; ++r) acc[r] += (s_s[r][pi] * vn) * val;
    }
    __syncthreads();
  }

  // reduce the PY position-slices, then write this split's partial state
  if (PY > 1) {
    if (py > 0) {
#pragma unroll
      for (int r = 0; r < kFgRMax; ++r) red_s[((py - 1) * kFgRMax + r) * DIM + e] = acc[r];
    }
    __syncthreads();
    if (py == 0) {
      for (int y = 1; y < PY; ++y)
#pragma unroll
        for (int r = 0; r < kFgRMax; ++r) acc[r] += red_s[((y - 1) * kFgRMax + r) * DIM + e];
    }
  }
  if (py == 0) {
    const int64_t n_rows = (int64_t)a.batch * a.n_q_heads;
    for (int r = 0; r < nr; ++r) {
      const int64_t row = (int64_t)b * a.n_q_heads + h0 + r;
      a.part_acc[((int64_t)split * n_rows + row) * DIM + e] = acc[r];
      if (e == 0) {
        a.part_m[(int64_t)split * n_rows + row] = m_s[r];
        a.part_l[(int64_t)split * n_rows + row] = l_s[r];
      }
    }
  }
}

// ---------------------------------------------------------------------------
// merge of partial states (split-K chunks or ranks)
// ---------------------------------------------------------------------------
template <typename T>
__global__ void merge_partials_kernel(const float* pm, int64_t sm, const float* pl,
                                      int64_t sl, const float* pacc, int64_t sa,
                                      int n_parts, int64_t n_rows,
                                      int dim, int rotate, SignMask signs, int finalize, T* out,
                                      int64_t out_row_stride, int64_t rows_per_batch,
                                      int64_t out_batch_stride, float* om, float* ol, float* oacc,
                                      const PeerGate gate) {
  __shared__ float sh[256];
  const int64_t row = blockIdx.x;
  const int e = threadIdx.x;
  // a decode kernel launched behind this merge with programmatic stream serialization may set up
  // now; it waits for this grid's completion before it reads the query or touches its workspace
  if (e == 0) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  bool gate_failed = false;
  // A merge that resets its gate is launched with programmatic stream serialization (see launch_merge):
  // it is resident early only so that the decode launch behind it may start; its own work begins once
  // the kernel in front of it has completed, like an ordinary launch (two merges that share a gate must
  // never wait on it at the same time).
  // (reset == 2: the flags are this merge's alone - one set per layer - so nothing has to be waited for
  // up front; the merge only must not complete before its predecessor, see the end of the kernel.)
  if (gate.flags != nullptr && gate.reset == 1) asm volatile("griddepcontrol.wait;" ::: "memory");
  if (gate.flags != nullptr) {
    // parts pushed by peer GPUs: one thread per rank waits for that rank's flag, bounded by a time
    // limit on the GPU-wide nanosecond timer (and by an iteration count as a second bound)
    __shared__ int failed_s;
    if (e == 0) failed_s = 0;
    __syncthreads();
    if (e < gate.n) {
      bool seen = false;
      unsigned long long t0;
      asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
      for (uint32_t it = 0; it < (1u << 28) && !seen; ++it) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(gate.flags + e) : "memory");
        seen = (int32_t)(v - gate.epoch) >= 0;
        if (!seen) {
          __nanosleep(50);
          unsigned long long t1;
          asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
          if (t1 - t0 > gate.limit_ns) break;
        }
      }
      if (!seen) {
        atomicExch(gate.status, 21 + e);
        failed_s = 1;
      }
    }
    __syncthreads();
    gate_failed = failed_s != 0;
    if (gate.reset) {
      // every block has to pass the gate before the flags go back to zero: the last one does it
      if (e == 0) {
        __threadfence();
        const int prev = atomicAdd(gate.done, 1);
        if (prev == (int)gridDim.x - 1) {
          for (int i = 0; i < gate.n; ++i)
            asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(gate.flags + i), "r"(0u) : "memory");
          *gate.done = 0;
        }
      }
    }
  }
  float m_star = -INFINITY;
  float l_star = 0.f, acc = 0.f;
  if (n_parts <= 16) {
    // few parts (ranks of a node, a handful of chunks): every load is issued before the first use,
    // so the kernel pays one trip to memory instead of one per part
    float mi[16], li[16], ai[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const bool on = i < n_parts;
      li[i] = on ? __ldcg(pl + (int64_t)i * sl + row) : 0.f;
      mi[i] = on ? __ldcg(pm + (int64_t)i * sm + row) : -INFINITY;
      ai[i] = on ? __ldcg(pacc + (int64_t)i * sa + row * dim + e) : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 16; ++i)
      if (li[i] > 0.f) m_star = fmaxf(m_star, mi[i]);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (!(li[i] > 0.f)) continue;   // empty or fully masked chunk merges as a no-op
      const float w = __expf(mi[i] - m_star);
      l_star += li[i] * w;
      acc += ai[i] * w;
    }
  } else {
    for (int i = 0; i < n_parts; ++i) {
      const float li = __ldcg(pl + (int64_t)i * sl + row);
      const float mi = __ldcg(pm + (int64_t)i * sm + row);
      if (li > 0.f) m_star = fmaxf(m_star, mi);
    }
    for (int i = 0; i < n_parts; ++i) {
      const float li = __ldcg(pl + (int64_t)i * sl + row);
      if (!(li > 0.f)) continue;   // empty or fully masked chunk merges as a no-op
      const float w = __expf(__ldcg(pm + (int64_t)i * sm + row) - m_star);
      l_star += li * w;
      acc += __ldcg(pacc + (int64_t)i * sa + row * dim + e) * w;
    }
  }
  if (!finalize) {
    oacc[row * dim + e] = acc;
    if (e == 0) {
      om[row] = m_star;
      ol[row] = l_star;
    }
    return;
  }
  float res = acc;
  if (rotate) {
    sh[e] = acc;
    __syncthreads();
    for (int hh = 1; hh < dim; hh <<= 1) {
      if ((e & hh) == 0) {
        float x = sh[e], y = sh[e + hh];
        sh[e] = x + y;
        sh[e + hh] = x - y;
      }
      __syncthreads();
    }
    res = sh[e] * sign_at(signs, e) * (1.0f / dim);
  }
  res = l_star > 0.f ? res / l_star : 0.f;
  if (gate_failed) res = __int_as_float(0x7fc00000);   // a rank never pushed: do not hand out a partial merge
  const int64_t bb = row / rows_per_batch, hh2 = row - bb * rows_per_batch;
  out[bb * out_batch_stride + hh2 * out_row_stride + e] = from_f32<T>(res);
  if (gate.flags != nullptr && gate.reset == 2) asm volatile("griddepcontrol.wait;" ::: "memory");
}

int launch_merge(const float* pm, int64_t sm, const float* pl, int64_t sl, const float* pacc,
                 int64_t sa, int n_parts, int64_t n_rows,
                 int dim, int rotate, const SignMask& signs, int finalize, void* out, int out_dtype,
                 int64_t out_row_stride, int64_t rows_per_batch, int64_t out_batch_stride,
                 float* om, float* ol, float* oacc, cudaStream_t st, const PeerGate* gate_in) {
  if (n_rows <= 0) return TQ_OK;
  PeerGate gate = {nullptr, 0, 0u, nullptr, 0, nullptr, 0ull};
  if (gate_in) gate = *gate_in;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)n_rows);
  cfg.blockDim = dim3(dim);
  cfg.stream = st;
  // A merge that resets its gate (the replayed, all-device-side exchange) is launched with programmatic
  // stream serialization: it becomes resident while the decode kernel in front of it runs, releases the
  // launch behind it at once (the next layer's decode, which depends on neither) and then waits for its
  // predecessor's completion before it touches the gate.  Every other merge is an ordinary launch.
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  if (gate.flags != nullptr && gate.reset) {
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  cudaError_t e;
#define TQ_MERGE(T)                                                                                        \
  e = cudaLaunchKernelEx(&cfg, merge_partials_kernel<T>, pm, sm, pl, sl, pacc, sa, n_parts, n_rows, dim, rotate, \
                         signs, finalize, (T*)out, out_row_stride, rows_per_batch, out_batch_stride, om, ol, \
                         oacc, gate)
  if (!finalize || out_dtype == TQ_F32) TQ_MERGE(float);
  else if (out_dtype == TQ_F16) TQ_MERGE(__half);
  else if (out_dtype == TQ_BF16) TQ_MERGE(__nv_bfloat16);
  else return set_error(TQ_ERR_BAD_ARG, "unknown dtype %d", out_dtype);
#undef TQ_MERGE
  if (e != cudaSuccess) return set_error(TQ_ERR_LAUNCH, "tq_merge_partials: %s", cudaGetErrorString(e));
  return check_launch("tq_merge_partials");
}

int launch_flash_generic(const FlashArgs& a, int splits, cudaStream_t st) {
  const int rgroups = (a.n_rep + kFgRMax - 1) / kFgRMax;
  const dim3 grid(splits, a.n_kv_heads * rgroups, a.batch);
  switch (a.dim) {
    case 32: flash_generic_kernel<1><<<grid, kFgThreads, 0, st>>>(a); break;
    case 64: flash_generic_kernel<2><<<grid, kFgThreads, 0, st>>>(a); break;
    case 128: flash_generic_kernel<4><<<grid, kFgThreads, 0, st>>>(a); break;
    default: flash_generic_kernel<8><<<grid, kFgThreads, 0, st>>>(a); break;
  }
  return check_launch("tq_flash_decode (generic)");
}

template <int BITS>
static int launch_scores_bits(const float* q_rot, const uint32_t* kp, int64_t khs, const float* kn,
                              int64_t knhs, int n_kv, int64_t seq, int n_rep, const Table16& cent,
                              int dim, float* out, cudaStream_t st) {
  const dim3 grid((unsigned)((seq + kScorePosPerBlock - 1) / kScorePosPerBlock), n_kv);
  const size_t sm = (size_t)n_rep * dim * sizeof(float);
  const float inv_dim = 1.0f / dim;
#define TQ_LAUNCH(EPL)                                                                        \
  prerot_scores_kernel<EPL, BITS><<<grid, kScoreWarps * 32, sm, st>>>(q_rot, kp, khs, kn, knhs, \
                                                                      seq, n_rep, cent, inv_dim, out)
  switch (dim) {
    case 32: TQ_LAUNCH(1); break;
    case 64: TQ_LAUNCH(2); break;
    case 128: TQ_LAUNCH(4); break;
    default: TQ_LAUNCH(8); break;
  }
#undef TQ_LAUNCH
  return check_launch("tq_prerot_qk_scores");
}

template <int BITS>
static int launch_packed_scores_bits(const float* q, const uint32_t* kp, int64_t khs,
                                     const float* kn, int64_t knhs, int n_heads, int64_t seq,
                                     const Table16& cs, const SignMask& sg, float s, int dim,
                                     float* out, cudaStream_t st) {
  const dim3 grid((unsigned)((seq + kScorePosPerBlock - 1) / kScorePosPerBlock), n_heads);
#define TQ_LAUNCH(EPL) \
  packed_scores_kernel<EPL, BITS><<<grid, kScoreWarps * 32, 0, st>>>(q, kp, khs, kn, knhs, seq, cs, sg, s, out)
  switch (dim) {
    case 32: TQ_LAUNCH(1); break;
    case 64: TQ_LAUNCH(2); break;
    case 128: TQ_LAUNCH(4); break;
    default: TQ_LAUNCH(8); break;
  }
#undef TQ_LAUNCH
  return check_launch("tq_packed_qk_scores");
}

static void fill_table(Table16* t, const float* host, int n) {
  for (int i = 0; i < 16; ++i) t->v[i] = (host && i < n) ? host[i] : 0.f;
}

static int sparse_v_splits(int64_t seq) {
  int64_t s = (seq + 511) / 512;
  return (int)(s < 1 ? 1 : (s > 256 ? 256 : s));
}

}  // namespace tq

using namespace tq;

extern "C" int tq_prerot_qk_scores(const float* q_rot, const uint32_t* k_packed,
                                   int64_t k_head_stride, const float* k_norms,
                                   int64_t kn_head_stride, int n_kv_heads, int64_t seq_len,
                                   const float* centroids_host, int dim, int bits, int n_rep,
                                   float* out, void* stream) {
  int rc = check_dim_bits(dim, bits, 256);
  if (rc) return rc;
  TQ_REQUIRE(n_kv_heads > 0 && n_rep > 0 && seq_len >= 0, TQ_ERR_BAD_ARG, "bad head / seq count");
  TQ_REQUIRE((size_t)n_rep * dim * 4 <= 40960, TQ_ERR_UNSUPPORTED, "n_rep * dim too large");
  TQ_REQUIRE(centroids_host != nullptr, TQ_ERR_BAD_ARG, "centroids pointer is NULL");
  if (seq_len == 0) return TQ_OK;
  TQ_REQUIRE(q_rot && k_packed && k_norms && out, TQ_ERR_BAD_ARG, "NULL tensor pointer");
  Table16 cent;
  fill_table(&cent, centroids_host, 1 << bits);
  cudaStream_t st = (cudaStream_t)stream;
  switch (bits) {
    case 1: return launch_scores_bits<1>(q_rot, k_packed, k_head_stride, k_norms, kn_head_stride, n_kv_heads, seq_len, n_rep, cent, dim, out, st);
    case 2: return launch_scores_bits<2>(q_rot, k_packed, k_head_stride, k_norms, kn_head_stride, n_kv_heads, seq_len, n_rep, cent, dim, out, st);
    case 3: return launch_scores_bits<3>(q_rot, k_packed, k_head_stride, k_norms, kn_head_stride, n_kv_heads, seq_len, n_rep, cent, dim, out, st);
    default: return launch_scores_bits<4>(q_rot, k_packed, k_head_stride, k_norms, kn_head_stride, n_kv_heads, seq_len, n_rep, cent, dim, out, st);
  }
}

extern "C" int tq_packed_qk_scores(const float* query, const uint32_t* k_packed,
                                   int64_t k_head_stride, const float* k_norms,
                                   int64_t kn_head_stride, int n_heads, int64_t seq_len,
                                   const float* centroids_host, const float* signs_host, int dim,
                                   int bits, float* out, void* stream) {
  int rc = check_dim_bits(dim, bits, 256);
  if (rc) return rc;
  TQ_REQUIRE(n_heads > 0 && seq_len >= 0, TQ_ERR_BAD_ARG, "bad head / seq count");
  TQ_REQUIRE(centroids_host != nullptr, TQ_ERR_BAD_ARG, "centroids pointer is NULL");
  if (seq_len == 0) return TQ_OK;
  TQ_REQUIRE(query && k_packed && k_norms && out, TQ_ERR_BAD_ARG, "NULL tensor pointer");
  SignMask sg;
  if ((rc = make_sign_mask(signs_host, dim, &sg))) return rc;
  const float s = (float)(1.0 / sqrt((double)dim));
  Table16 cs;
  for (int i = 0; i < 16; ++i) {
    volatile float v = (i < (1 << bits)) ? centroids_host[i] * s : 0.f;
    cs.v[i] = v;
  }
  cudaStream_t st = (cudaStream_t)stream;
  switch (bits) {
    case 1: return launch_packed_scores_bits<1>(query, k_packed, k_head_stride, k_norms, kn_head_stride, n_heads, seq_len, cs, sg, s, dim, out, st);
    case 2: return launch_packed_scores_bits<2>(query, k_packed, k_head_stride, k_norms, kn_head_stride, n_heads, seq_len, cs, sg, s, dim, out, st);
    case 3: return launch_packed_scores_bits<3>(query, k_packed, k_head_stride, k_norms, kn_head_stride, n_heads, seq_len, cs, sg, s, dim, out, st);
    default: return launch_packed_scores_bits<4>(query, k_packed, k_head_stride, k_norms, kn_head_stride, n_heads, seq_len, cs, sg, s, dim, out, st);
  }
}

extern "C" size_t tq_sparse_v_workspace_bytes(int n_q_heads, int64_t seq_len, int dim) {
  if (n_q_heads <= 0 || dim <= 0 || seq_len < 0) return 0;
  return (size_t)sparse_v_splits(seq_len) * n_q_heads * dim * sizeof(float);
}

extern "C" int tq_sparse_v_matvec(const float* weights, int64_t w_head_stride,
                                  const uint32_t* v_packed, int64_t v_head_stride,
                                  const float* v_norms, int64_t vn_head_stride, int n_kv_heads,
                                  int64_t seq_len, const float* centroids_host,
                                  const float* signs_host, int dim, int bits, float threshold,
                                  int n_rep, float* out, void* workspace, size_t workspace_bytes,
                                  void* stream) {
  if (dim <= 0 || (dim & (dim - 1)))
    return set_error(TQ_ERR_BAD_DIM, "dim must be a power of 2, got %d", dim);
  if (dim > 256)
    return set_error(TQ_ERR_BAD_DIM, "dim > 256 not supported by threadgroup layout, got %d", dim);
  int rc = check_dim_bits(dim, bits, 256);
  if (rc) return rc;
  TQ_REQUIRE(n_kv_heads > 0 && n_rep > 0 && seq_len >= 0, TQ_ERR_BAD_ARG, "bad head / seq count");
  TQ_REQUIRE(centroids_host != nullptr, TQ_ERR_BAD_ARG, "centroids pointer is NULL");
  TQ_REQUIRE(out != nullptr, TQ_ERR_BAD_ARG, "NULL output pointer");
  TQ_REQUIRE(seq_len == 0 || (weights && v_packed && v_norms), TQ_ERR_BAD_ARG, "NULL tensor pointer");
  const int n_q = n_kv_heads * n_rep;
  const size_t need = tq_sparse_v_workspace_bytes(n_q, seq_len, dim);
  TQ_REQUIRE(workspace && workspace_bytes >= need, TQ_ERR_WORKSPACE,
             "workspace of %zu bytes required, got %zu", need, workspace_bytes);
  SignMask sg;
  if ((rc = make_sign_mask(signs_host, dim, &sg))) return rc;
  Table16 cent;
  fill_table(&cent, centroids_host, 1 << bits);
  const int splits = sparse_v_splits(seq_len);
  const int64_t chunk = (seq_len + splits - 1) / splits;
  const float thr = threshold > 0.f ? threshold : 0.f;
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid(splits, n_kv_heads, (n_rep + kSvRMax - 1) / kSvRMax);
  float* ws = (float*)workspace;
#define TQ_LAUNCH(B)                                                                             \
  sparse_v_partial_kernel<B><<<grid, 256, 0, st>>>(weights, w_head_stride, v_packed, v_head_stride, \
                                                   v_norms, vn_head_stride, seq_len,               \
                                                   chunk > 0 ? chunk : 1, dim, n_rep, thr, cent, ws, n_q)
  switch (bits) {
    case 1: TQ_LAUNCH(1); break;
    case 2: TQ_LAUNCH(2); break;
    case 3: TQ_LAUNCH(3); break;
    default: TQ_LAUNCH(4); break;
  }
#undef TQ_LAUNCH
  if ((rc = check_launch("tq_sparse_v_matvec (partial)"))) return rc;
  sparse_v_finish_kernel<<<n_q, dim, 0, st>>>(ws, splits, n_q, dim, sg, 1.0f / dim, out);
  return check_launch("tq_sparse_v_matvec (finish)");
}

extern "C" int tq_merge_partials(const float* part_m, int64_t m_part_stride, const float* part_l,
                                 int64_t l_part_stride, const float* part_acc,
                                 int64_t acc_part_stride, int n_parts, int64_t n_rows, int dim,
                                 const float* v_signs_host, void* out, int out_dtype,
                                 int64_t out_row_stride, void* stream) {
  TQ_REQUIRE(dim >= 32 && dim <= 256 && !(dim & (dim - 1)), TQ_ERR_BAD_DIM,
             "dim must be a power of 2 in [32, 256], got %d", dim);
  TQ_REQUIRE(n_parts > 0 && n_rows >= 0, TQ_ERR_BAD_ARG, "bad part / row count");
  if (n_rows == 0) return TQ_OK;
  TQ_REQUIRE(part_m && part_l && part_acc && out, TQ_ERR_BAD_ARG, "NULL tensor pointer");
  SignMask sg = {};
  int rc;
  if (v_signs_host && (rc = make_sign_mask(v_signs_host, dim, &sg))) return rc;
  return launch_merge(part_m, m_part_stride, part_l, l_part_stride, part_acc, acc_part_stride,
                      n_parts, n_rows, dim, v_signs_host != nullptr, sg, 1, out, out_dtype,
                      out_row_stride, n_rows, 0, nullptr, nullptr, nullptr, (cudaStream_t)stream);
}

extern "C" int tq_merge_partials_after_peers(void* flags, int n_ranks, uint32_t epoch, int* status, int reset_flags,
                                             const float* part_m, int64_t m_part_stride, const float* part_l,
                                             int64_t l_part_stride, const float* part_acc,
                                             int64_t acc_part_stride, int n_parts, int64_t n_rows, int dim,
                                             const float* v_signs_host, void* out, int out_dtype,
                                             int64_t out_row_stride, void* stream) {
  TQ_REQUIRE(dim >= 32 && dim <= 256 && !(dim & (dim - 1)), TQ_ERR_BAD_DIM,
             "dim must be a power of 2 in [32, 256], got %d", dim);
  TQ_REQUIRE(n_parts > 0 && n_rows >= 0, TQ_ERR_BAD_ARG, "bad part / row count");
  TQ_REQUIRE(flags && status && n_ranks >= 1 && n_ranks <= dim, TQ_ERR_BAD_ARG, "bad flag array");
  if (n_rows == 0) return TQ_OK;
  TQ_REQUIRE(part_m && part_l && part_acc && out, TQ_ERR_BAD_ARG, "NULL tensor pointer");
  SignMask sg = {};
  int rc;
  if (v_signs_host && (rc = make_sign_mask(v_signs_host, dim, &sg))) return rc;
  // status[0]: give-up code; status[1]: blocks past the gate (reset_flags only), zero between calls
  TQ_REQUIRE(reset_flags >= 0 && reset_flags <= 2, TQ_ERR_BAD_ARG, "reset_flags must be 0, 1 or 2");
  // blocks past the gate are counted in status[1] (merges that follow one another) or, for a merge that
  // may run beside others (reset_flags 2), in the word behind its own flag words
  int* done = reset_flags == 2 ? reinterpret_cast<int*>(static_cast<uint32_t*>(flags) + n_ranks) : status + 1;
  const PeerGate gate = {static_cast<uint32_t*>(flags), n_ranks, epoch, status, reset_flags, done,
                         peer_wait_limit_ns()};
  return launch_merge(part_m, m_part_stride, part_l, l_part_stride, part_acc, acc_part_stride,
                      n_parts, n_rows, dim, v_signs_host != nullptr, sg, 1, out, out_dtype,
                      out_row_stride, n_rows, 0, nullptr, nullptr, nullptr, (cudaStream_t)stream, &gate);
}

// ---------------------------------------------------------------------------
// tq_sparse_v_matvec_noalloc: the same two kernels as tq_sparse_v_matvec, with
// the partial-sum scratch taken from a fixed array inside the library instead of
// a caller-supplied workspace.  It exists for callers that are not in a position
// to allocate device memory at all: code running under a serving framework that
// owns every byte of device memory through its own arena and forbids plugins
// from calling cudaMalloc, bindings from languages that can pass pointers they
// were given but have no allocator of their own, and call sites where an
// allocation would stall the device (cudaMalloc synchronises) in the middle of
// a latency-critical decode loop.
//
// The array lives in every process that loads the library, on every GPU the
// process touches, until exit - hence the modest, fixed size.  All calls share
// it: two calls that overlap on the GPU (different streams, or different
// threads) race on it and must be serialised by the caller.  It keeps whatever
// the previous call left behind; that is harmless here because the first kernel
// overwrites every word the second kernel reads, so nothing has to be cleared.
// ---------------------------------------------------------------------------
#define TQ_SPARSE_V_STATIC_BYTES (4u << 20)
static __device__ __align__(256) unsigned char g_sparse_v_scratch[TQ_SPARSE_V_STATIC_BYTES];

#include <mutex>

// In host code the array's name is only a handle; the device address has to be
// looked up, per device, with that device current.  Done on the first call that
// runs on a device (so that call should come before any stream capture).
static int sparse_v_static_scratch(float** out) {
  static std::mutex mu;
  static float* ptrs[64] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64)
    return set_error(TQ_ERR_LAUNCH, "cudaGetDevice failed or device index %d out of range: %s", dev,
                     cudaGetErrorString(e));
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_sparse_v_scratch);
    if (e != cudaSuccess || p == nullptr)
      return set_error(TQ_ERR_LAUNCH, "cudaGetSymbolAddress(scratch) on device %d: %s", dev,
                       cudaGetErrorString(e));
    ptrs[dev] = reinterpret_cast<float*>(p);
  }
  *out = ptrs[dev];
  return TQ_OK;
}

extern "C" size_t tq_sparse_v_noalloc_max_bytes(void) { return TQ_SPARSE_V_STATIC_BYTES; }

extern "C" int tq_sparse_v_matvec_noalloc(const float* weights, int64_t w_head_stride,
                                          const uint32_t* v_packed, int64_t v_head_stride,
                                          const float* v_norms, int64_t vn_head_stride,
                                          int n_kv_heads, int64_t seq_len,
                                          const float* centroids_host, const float* signs_host,
                                          int dim, int bits, float threshold, int n_rep,
                                          float* out, void* stream) {
  if (dim <= 0 || (dim & (dim - 1)))
    return set_error(TQ_ERR_BAD_DIM, "dim must be a power of 2, got %d", dim);
  if (dim > 256)
    return set_error(TQ_ERR_BAD_DIM, "dim > 256 not supported by threadgroup layout, got %d", dim);
  int rc = check_dim_bits(dim, bits, 256);
  if (rc) return rc;
  TQ_REQUIRE(n_kv_heads > 0 && n_rep > 0 && seq_len >= 0, TQ_ERR_BAD_ARG, "bad head / seq count");
  TQ_REQUIRE(centroids_host != nullptr, TQ_ERR_BAD_ARG, "centroids pointer is NULL");
  TQ_REQUIRE(out != nullptr, TQ_ERR_BAD_ARG, "NULL output pointer");
  TQ_REQUIRE(seq_len == 0 || (weights && v_packed && v_norms), TQ_ERR_BAD_ARG, "NULL tensor pointer");
  const int n_q = n_kv_heads * n_rep;
  const size_t need = tq_sparse_v_workspace_bytes(n_q, seq_len, dim);
  TQ_REQUIRE(need <= TQ_SPARSE_V_STATIC_BYTES, TQ_ERR_WORKSPACE,
             "this call needs %zu bytes of scratch but the built-in array holds %u; use "
             "tq_sparse_v_matvec with a caller-provided workspace for this size",
             need, (unsigned)TQ_SPARSE_V_STATIC_BYTES);
  float* ws = nullptr;
  if ((rc = sparse_v_static_scratch(&ws))) return rc;
  SignMask sg;
  if ((rc = make_sign_mask(signs_host, dim, &sg))) return rc;
  Table16 cent;
  fill_table(&cent, centroids_host, 1 << bits);
  const int splits = sparse_v_splits(seq_len);
  const int64_t chunk = (seq_len + splits - 1) / splits;
  const float thr = threshold > 0.f ? threshold : 0.f;
  cudaStream_t st = (cudaStream_t)stream;
  const dim3 grid(splits, n_kv_heads, (n_rep + kSvRMax - 1) / kSvRMax);
#define TQ_LAUNCH(B)                                                                             \
  sparse_v_partial_kernel<B><<<grid, 256, 0, st>>>(weights, w_head_stride, v_packed, v_head_stride, \
                                                   v_norms, vn_head_stride, seq_len,               \
                                                   chunk > 0 ? chunk : 1, dim, n_rep, thr, cent, ws, n_q)
  switch (bits) {
    case 1: TQ_LAUNCH(1); break;
    case 2: TQ_LAUNCH(2); break;
    case 3: TQ_LAUNCH(3); break;
    default: TQ_LAUNCH(4); break;
  }
#undef TQ_LAUNCH
  if ((rc = check_launch("tq_sparse_v_matvec_noalloc (partial)"))) return rc;
  sparse_v_finish_kernel<<<n_q, dim, 0, st>>>(ws, splits, n_q, dim, sg, 1.0f / dim, out);
  return check_launch("tq_sparse_v_matvec_noalloc (finish)");
}
