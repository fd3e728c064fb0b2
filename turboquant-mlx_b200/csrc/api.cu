// Error reporting, version and the small host-side parameter builders.
#include <math.h>
#include <stdarg.h>
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace tq {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  cudaError_t e = cudaPeekAtLastError();
  if (e != cudaSuccess) {
    return set_error(TQ_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  }
  return TQ_OK;
}

int make_sign_mask(const float* signs, int dim, SignMask* out) {
  memset(out, 0, sizeof(*out));
  if (!signs) return set_error(TQ_ERR_BAD_ARG, "signs pointer is NULL");
  for (int e = 0; e < dim; ++e) {
    if (signs[e] == -1.0f) {
      out->w[e >> 5] |= 1u << (e & 31);
    } else if (signs[e] != 1.0f) {
      return set_error(TQ_ERR_BAD_ARG, "signs[%d] = %g, every sign must be +1 or -1", e,
                       (double)signs[e]);
    }
  }
  return TQ_OK;
}

int check_dim_bits(int dim, int bits, int max_dim) {
  if (dim < 32 || dim > max_dim || (dim & (dim - 1)))
    return set_error(TQ_ERR_BAD_DIM, "dim must be a power of 2 in [32, %d], got %d", max_dim, dim);
  if (bits < 1 || bits > 4)
    return set_error(TQ_ERR_BAD_BITS, "Unsupported bit width: %d. Use 1-4.", bits);
  return TQ_OK;
}

static inline float next_up(float x) { return nextafterf(x, INFINITY); }
static inline float next_down(float x) { return nextafterf(x, -INFINITY); }

void make_raw_thresholds(const float* b, int n, int dim, Table16* out) {
  const float s = (float)(1.0 / sqrt((double)dim));
  for (int i = 0; i < 16; ++i) out->v[i] = INFINITY;
  for (int i = 0; i < n; ++i) {
    const float bi = b[i];
    volatile float y = bi;
    // f(y) = (y * s) / s in float32, evaluated with IEEE single operations.
    auto f = [s](float v) {
      volatile float r = v * s;
      volatile float z = r / s;
      return (float)z;
    };
    int guard = 0;
    while (f(y) <= bi && guard++ < 64) y = next_up(y);      // first y with f(y) > b
    guard = 0;
    while (f(y) > bi && guard++ < 128) y = next_down(y);    // largest y with f(y) <= b
    out->v[i] = y;
  }
}

int num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace tq

extern "C" int tq_version(void) { return 100; }  // 0.1.0
extern "C" const char* tq_last_error_string(void) { return tq::g_err; }
