// minGRU: a gated recurrence whose gates read only the current token.
//
//   z_t = sigmoid(a_t)            a, u, g: three projections of the token (biases added by the projection)
//   c_t = u_t + 1/2  (u_t >= 0),  sigmoid(u_t)  (u_t < 0)
//   S_t = (1 - z_t) S_(t-1) + z_t c_t          element by element, float32, from the sequence's state
//   y_t = S_t * g_t * sigmoid(g_t)
//
// One thread owns one channel of one batch row and walks the row's tokens of this step in order: the state is read
// from and written back to the row's slot, so a sequence cut into steps in any way gives the same sums (up to
// rounding, see below).  Loads of the next tokens do not depend on S and are issued ahead of the chain of multiply-adds.
//
// Rows that bring many tokens (prompts) are cut into chunks of RC_CHUNK tokens that run side by side.  The
// recurrence is linear in S: over a chunk, S_out = A S_in + B with A = prod (1 - z_t) and B the chunk's own scan from
// zero.  A first kernel leaves (A, B) per chunk and channel; a second one folds the (A, B) of the chunks before its
// own, in order, into its starting state and then walks its chunk as above.
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

constexpr int RC_CHUNK = 32;

// Chunk j of batch row b has a place of its own among floor(T / RC_CHUNK) + B + 1 places: rows are packed one after
// another, so floor(first token / RC_CHUNK) + b + j never meets another row's.
__device__ inline int rc_chunk_place(int t0, int b, int j) { return t0 / RC_CHUNK + b + j; }

// The chunk kernels.  FAST (16-bit projections, whose own rounding is 2^-9): the exponentials and reciprocals of the
// gates by the short instructions (2^-21 or so); float32 projections take the exact ones.
template <bool FAST>
__device__ inline float rc_sig(float v) {
  return FAST ? __fdividef(1.0f, 1.0f + __expf(-v)) : 1.0f / (1.0f + expf(-v));
}

template <bool FAST>
__global__ void __launch_bounds__(128)
mingru_chunk_kernel(const void* zug, int zug_dtype, float* ab, const int* __restrict__ row_start, int width, int places) {
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.z, j = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int t0 = __ldcg(row_start + b), t1 = __ldcg(row_start + b + 1);
  const int a0 = t0 + j * RC_CHUNK;
  if (c >= width || a0 + RC_CHUNK >= t1) return;       // the row's last chunk has nobody after it
  const int64_t ld = 3 * (int64_t)width;
  float A = 1.0f, Bv = 0.0f;
  for (int t = a0; t < a0 + RC_CHUNK; t += RC_AHEAD) {
    float a[RC_AHEAD], u[RC_AHEAD];
#pragma unroll
    for (int i = 0; i < RC_AHEAD; ++i) {
      a[i] = rc_load(zug, zug_dtype, (int64_t)(t + i) * ld + c);
      u[i] = rc_load(zug, zug_dtype, (int64_t)(t + i) * ld + c + width);
    }
#pragma unroll
    for (int i = 0; i < RC_AHEAD; ++i) {
      const float z = rc_sig<FAST>(a[i]);
      const float cand = u[i] >= 0.0f ? u[i] + 0.5f : rc_sig<FAST>(u[i]);
      A *= 1.0f - z;
      Bv = fmaf(z, cand, (1.0f - z) * Bv);
    }
  }
  const int64_t at = (int64_t)rc_chunk_place(t0, b, j) * width + c;
  ab[at] = A;
  ab[(int64_t)places * width + at] = Bv;
}

template <bool FAST>
__global__ void __launch_bounds__(128)
mingru_chunk_scan_kernel(const void* zug, int zug_dtype, void* y, int y_dtype, float* state, const float* ab,
                         const int* __restrict__ slot_ids, const int* __restrict__ row_start, int width, int places) {
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.z, j = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int t0 = __ldcg(row_start + b), t1 = __ldcg(row_start + b + 1);
  const int a0 = t0 + j * RC_CHUNK;
  if (c >= width || a0 >= t1) return;
  float* sp = state + (int64_t)__ldcg(slot_ids + b) * width + c;
  float S = __ldcg(sp);
  for (int i = 0; i < j; ++i) {                        // the chunks before this one, in order
    const int64_t at = (int64_t)rc_chunk_place(t0, b, i) * width + c;
    S = fmaf(__ldcg(ab + at), S, __ldcg(ab + (int64_t)places * width + at));
  }
  const int a1 = min(a0 + RC_CHUNK, t1);
  const int64_t ld = 3 * (int64_t)width;
  for (int t = a0; t < a1; t += RC_AHEAD) {
    float a[RC_AHEAD], u[RC_AHEAD], g[RC_AHEAD];
#pragma unroll
    for (int i = 0; i < RC_AHEAD; ++i) {
      const int64_t at = (int64_t)(t + i < a1 ? t + i : t) * ld + c;
      a[i] = rc_load(zug, zug_dtype, at);
      u[i] = rc_load(zug, zug_dtype, at + width);
      g[i] = rc_load(zug, zug_dtype, at + 2 * (int64_t)width);
    }
#pragma unroll
    for (int i = 0; i < RC_AHEAD; ++i) {
      if (t + i < a1) {
        const float z = rc_sig<FAST>(a[i]);
        const float cand = u[i] >= 0.0f ? u[i] + 0.5f : rc_sig<FAST>(u[i]);
        S = fmaf(z, cand, (1.0f - z) * S);
        const float o = S * g[i] * rc_sig<FAST>(g[i]);
        const int64_t oi = (int64_t)(t + i) * width + c;
        if (y_dtype == DT_F32) static_cast<float*>(y)[oi] = o;
        else static_cast<__nv_bfloat16*>(y)[oi] = __float2bfloat16_rn(o);
      }
    }
  }
  if (a1 == t1) *sp = S;                               // the row's last chunk leaves the state
}

}  // namespace exl3

using namespace exl3;

extern "C" size_t exl3_mingru_scratch_bytes(int B, int T, int width, int max_new) {
  if (max_new <= 4 * RC_CHUNK) return 0;                       // few tokens: one thread walks a row's channel
  return 2 * (size_t)(T / RC_CHUNK + B + 1) * width * sizeof(float);
}

extern "C" int exl3_mingru_scan(const void* zug, int zug_dtype, void* y, int y_dtype, float* state,
                                const int* slot_ids, const int* row_start, int B, int T, int width, int max_new,
                                float* scratch, size_t scratch_bytes, cudaStream_t stream) {
  if (B == 0 || T == 0) return 0;
  if (B < 0 || T < 0 || width < 1 || B > 65535) {
    set_error("mingru_scan: bad sizes rows=%d tokens=%d width=%d", B, T, width);
    return ERR_BAD_ARGUMENT;
  }
  if (max_new > 4 * RC_CHUNK) {
    // prompts: chunks side by side (see the top of the file)
    const int chunks = ceil_div(max_new, RC_CHUNK), places = T / RC_CHUNK + B + 1;
    if (scratch == nullptr || exl3_mingru_scratch_bytes(B, T, width, max_new) > scratch_bytes || chunks > 65535) {
      set_error("mingru_scan: scratch of %zu bytes is too small for %d tokens", scratch_bytes, T);
      return ERR_SCRATCH;
    }
    dim3 grid(ceil_div(width, 128), chunks, B);
    if (zug_dtype == DT_BF16)
      launch_pdl(mingru_chunk_kernel<true>, grid, dim3(128), 0, stream, zug, zug_dtype, scratch, row_start, width, places);
    else
      launch_pdl(mingru_chunk_kernel<false>, grid, dim3(128), 0, stream, zug, zug_dtype, scratch, row_start, width, places);
    int rc = launch_status("mingru_chunk");
    if (rc) return rc;
    if (zug_dtype == DT_BF16)
      launch_pdl(mingru_chunk_scan_kernel<true>, grid, dim3(128), 0, stream, zug, zug_dtype, y, y_dtype, state,
                 (const float*)scratch, slot_ids, row_start, width, places);
    else
      launch_pdl(mingru_chunk_scan_kernel<false>, grid, dim3(128), 0, stream, zug, zug_dtype, y, y_dtype, state,
                 (const float*)scratch, slot_ids, row_start, width, places);
    return launch_status("mingru_chunk_scan");
  }
  launch_pdl(mingru_scan_kernel, dim3(ceil_div(width, 128), B), dim3(128), 0, stream, zug, zug_dtype, y, y_dtype, state,
             slot_ids, row_start, width);
  return launch_status("mingru_scan");
}
