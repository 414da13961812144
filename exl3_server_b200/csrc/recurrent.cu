// minGRU: a gated recurrence whose gates read only the current token.
//
//   z_t = sigmoid(a_t)            a, u, g: three projections of the token (biases added by the projection)
//   c_t = u_t + 1/2  (u_t >= 0),  sigmoid(u_t)  (u_t < 0)
//   S_t = (1 - z_t) S_(t-1) + z_t c_t          element by element, float32, from the sequence's state
//   y_t = S_t * g_t * sigmoid(g_t)
//
// One thread owns one channel of one batch row and walks the row's tokens of this step in order: the state is read
// from and written back to the row's slot, so a sequence cut into steps in any way gives the same sums.  Loads of
// the next tokens do not depend on S and are issued ahead of the chain of multiply-adds.
#include "api.h"
#include "common.cuh"

namespace exl3 {

__device__ inline float rc_load(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? __ldcg(static_cast<const float*>(p) + i)
                         : __bfloat162float(__ldcg(static_cast<const __nv_bfloat16*>(p) + i));
}
__device__ inline float rc_sigmoid(float v) { return 1.0f / (1.0f + expf(-v)); }

constexpr int RC_AHEAD = 8;

__global__ void __launch_bounds__(128)
mingru_scan_kernel(const void* zug, int zug_dtype, void* y, int y_dtype, float* state, const int* __restrict__ slot_ids,
                   const int* __restrict__ row_start, int width) {
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= width) return;
  const int t0 = __ldcg(row_start + b), t1 = __ldcg(row_start + b + 1);
  float* sp = state + (int64_t)__ldcg(slot_ids + b) * width + c;
  float S = __ldcg(sp);
  const int64_t ld = 3 * (int64_t)width;
  for (int t = t0; t < t1; t += RC_AHEAD) {
    float a[RC_AHEAD], u[RC_AHEAD], g[RC_AHEAD];
#pragma unroll
    for (int i = 0; i < RC_AHEAD; ++i) {
      const bool in = t + i < t1;
      const int64_t at = (int64_t)(in ? t + i : t) * ld + c;
      a[i] = rc_load(zug, zug_dtype, at);
      u[i] = rc_load(zug, zug_dtype, at + width);
      g[i] = rc_load(zug, zug_dtype, at + 2 * (int64_t)width);
    }
#pragma unroll
    for (int i = 0; i < RC_AHEAD; ++i) {
      if (t + i < t1) {
        const float z = rc_sigmoid(a[i]);
        const float cand = u[i] >= 0.0f ? u[i] + 0.5f : rc_sigmoid(u[i]);
        S = fmaf(z, cand, (1.0f - z) * S);
        const float o = S * g[i] * rc_sigmoid(g[i]);
        const int64_t oi = (int64_t)(t + i) * width + c;
        if (y_dtype == DT_F32) static_cast<float*>(y)[oi] = o;
        else static_cast<__nv_bfloat16*>(y)[oi] = __float2bfloat16_rn(o);
      }
    }
  }
  *sp = S;
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_mingru_scan(const void* zug, int zug_dtype, void* y, int y_dtype, float* state,
                                const int* slot_ids, const int* row_start, int B, int T, int width, int max_new,
                                cudaStream_t stream) {
  if (B == 0 || T == 0) return 0;
  if (B < 0 || T < 0 || width < 1 || B > 65535) {
    set_error("mingru_scan: bad sizes rows=%d tokens=%d width=%d", B, T, width);
    return ERR_BAD_ARGUMENT;
  }
  (void)max_new;
  launch_pdl(mingru_scan_kernel, dim3(ceil_div(width, 128), B), dim3(128), 0, stream, zug, zug_dtype, y, y_dtype, state,
             slot_ids, row_start, width);
  return launch_status("mingru_scan");
}
