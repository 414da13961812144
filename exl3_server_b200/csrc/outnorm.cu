// Parts of a layer whose norm sits on the sublayer's OUTPUT, and the xIELU activation.
//
//   norm_add:  h += y * rsqrt(mean(y^2) + eps) * w        (the residual sum, float32)
//              x  = h in the activation type                (what the next sublayer's projections read)
//   xielu:     a(z) = softplus(p) z^2 + z / 2                          for z > 0
//                     (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2     for z <= 0
//
// Statistics, the sum and the activation are float32 whatever the element types around them.
#include "api.h"
#include "common.cuh"

namespace exl3 {

__device__ inline float on_load_any(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? static_cast<const float*>(p)[i]
                         : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}
// for data that an earlier kernel of the same step wrote: through L2 (see load_vec_cg in common.cuh)
__device__ inline float on_load_act(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? __ldcg(static_cast<const float*>(p) + i)
                         : __bfloat162float(__ldcg(static_cast<const __nv_bfloat16*>(p) + i));
}
__device__ inline void on_store_any(void* p, int dtype, int64_t i, float v) {
  if (dtype == DT_F32) static_cast<float*>(p)[i] = v;
  else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

constexpr int NA_THREADS = 256;
constexpr int NA_KEEP = 8;                       // values of y a thread keeps in registers: rows up to 2048 are read once

__global__ void __launch_bounds__(NA_THREADS)
norm_add_kernel(float* h, const void* y, int y_dtype, const void* __restrict__ w, int w_dtype, float eps, void* x,
                int x_dtype, int H) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int64_t base = (int64_t)blockIdx.x * H;
  if (y == nullptr) {
    if (x) for (int c = threadIdx.x; c < H; c += NA_THREADS) on_store_any(x, x_dtype, base + c, __ldcg(h + base + c));
    return;
  }
  float keep[NA_KEEP];
  float ss = 0.0f;
#pragma unroll
  for (int p = 0; p < NA_KEEP; ++p) {
    const int c = p * NA_THREADS + threadIdx.x;
    keep[p] = c < H ? on_load_act(y, y_dtype, base + c) : 0.0f;
    ss += keep[p] * keep[p];
  }
  for (int c = NA_KEEP * NA_THREADS + threadIdx.x; c < H; c += NA_THREADS) {
    const float v = on_load_act(y, y_dtype, base + c);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  const float inv = 1.0f / sqrtf(ss / (float)H + eps);
#pragma unroll
  for (int p = 0; p < NA_KEEP; ++p) {
    const int c = p * NA_THREADS + threadIdx.x;
    if (c < H) {
      const float v = __ldcg(h + base + c) + keep[p] * inv * on_load_any(w, w_dtype, c);
      h[base + c] = v;
      if (x) on_store_any(x, x_dtype, base + c, v);
    }
  }
  for (int c = NA_KEEP * NA_THREADS + threadIdx.x; c < H; c += NA_THREADS) {
    const float v = __ldcg(h + base + c) + on_load_act(y, y_dtype, base + c) * inv * on_load_any(w, w_dtype, c);
    h[base + c] = v;
    if (x) on_store_any(x, x_dtype, base + c, v);
  }
}

__device__ inline float softplus_f(float v) { return v > 20.0f ? v : log1pf(expf(v)); }

__global__ void xielu_kernel(const void* z, int z_dtype, const void* __restrict__ pq, int pq_dtype, void* out,
                             int out_dtype, int64_t n) {
  pdl_wait();
  pdl_trigger();
  const float ap = softplus_f(on_load_any(pq, pq_dtype, 0));
  const float an = 0.5f + softplus_f(on_load_any(pq, pq_dtype, 1));
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const float v = on_load_act(z, z_dtype, i);
    const float r = v > 0.0f ? fmaf(ap * v, v, 0.5f * v) : fmaf(an, expm1f(v) - v, 0.5f * v);
    on_store_any(out, out_dtype, i, r);
  }
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_norm_add(float* h, const void* y, int y_dtype, const void* w, int w_dtype, float eps, void* x,
                             int x_dtype, int T, int H, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || H < 1 || (y != nullptr && w == nullptr) || (y == nullptr && x == nullptr)) {
    set_error("norm_add: bad arguments T=%d H=%d", T, H);
    return ERR_BAD_ARGUMENT;
  }
  launch_pdl(norm_add_kernel, dim3(T), dim3(NA_THREADS), 0, stream, h, y, y_dtype, w, w_dtype, eps, x, x_dtype, H);
  return launch_status("norm_add");
}

extern "C" int exl3_xielu(const void* z, int z_dtype, const void* pq, int pq_dtype, void* out, int out_dtype,
                          int64_t n, cudaStream_t stream) {
  if (n == 0) return 0;
  if (n < 0) { set_error("xielu: bad size"); return ERR_BAD_ARGUMENT; }
  int64_t blocks = (n + 255) / 256;
  if (blocks > 148 * 32) blocks = 148 * 32;
  launch_pdl(xielu_kernel, dim3((unsigned)blocks), dim3(256), 0, stream, z, z_dtype, pq, pq_dtype, out, out_dtype, n);
  return launch_status("xielu");
}
