// Latent attention: queries and keys/values go through low-rank latents, and the cache keeps one row per token
// that every head reads: [ c (kv_rank, normed) | rotated key part (rot_dim) ].
//
//   c_q = rmsnorm(W_dq x) * w_q          q_h = W_uq,h c_q = [ q_h^n (dim) | q_h^r (rot_dim) ]
//   [c' | k'] = W_dkv x                  c = rmsnorm(c') * w_kv,  k^r = rope(k')
//   score_h(i, j) = ( q_h^n(i) . W_uk,h c(j) + rope(q_h^r(i)) . k^r(j) ) * scale
//   o_h(i) = sigmoid(w_g,h . x(i)) * W_uv,h sum_j softmax_j(score_h(i, .)) c(j)
//
// Since W_uk,h c(j) is linear in c(j), the key side of the score is (W_uk,h^T q_h^n(i)) . c(j): the query is carried
// into the latent space once per token and head (head_gemm below), attention then runs over the cached rows as
// keys of kv_rank + rot_dim features whose first kv_rank features are also the values, and W_uv,h is applied to
// the attention's output (head_gemm again, with the gate as a factor).  Nothing per head is ever cached or
// recomputed for old tokens.
//
// latent_prep does everything between the joint input projection and the rest: both norms, the rotation of the
// shared key part, the cache write and the gate.
#include "api.h"
#include "common.cuh"

namespace exl3 {

__device__ inline float lt_load_w(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? static_cast<const float*>(p)[i]
                         : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ inline float lt_load(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? __ldcg(static_cast<const float*>(p) + i)
                         : __bfloat162float(__ldcg(static_cast<const __nv_bfloat16*>(p) + i));
}
__device__ inline void lt_store(void* p, int dtype, int64_t i, float v) {
  if (dtype == DT_F32) static_cast<float*>(p)[i] = v;
  else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

__global__ void __launch_bounds__(128)
latent_prep_kernel(const void* a, int a_dtype, int lda, int q_off, int q_rank, const void* __restrict__ wq, int wq_dtype,
                   int kv_off, int kv_rank, int rot_dim, const void* __restrict__ wkv, int wkv_dtype, int g_off, int heads,
                   float eps, const float* __restrict__ inv_freq, const float* __restrict__ inv_freq_lo, int rot,
                   const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, const int* __restrict__ block_table,
                   int bt_stride, int page, void* pool, int pool_dtype, int kv_row, int rank_pad, void* cq, int cq_dtype,
                   float* gate) {
  __shared__ float red[32];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int64_t row = (int64_t)t * lda;
  // the query latent
  float ss = 0.0f;
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
    const float v = lt_load(a, a_dtype, row + q_off + i);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  float inv = 1.0f / sqrtf(ss / (float)q_rank + eps);
  for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
    lt_store(cq, cq_dtype, (int64_t)t * q_rank + i, lt_load(a, a_dtype, row + q_off + i) * inv * lt_load_w(wq, wq_dtype, i));
  // the gates
  for (int i = threadIdx.x; i < heads; i += blockDim.x)
    gate[(int64_t)t * heads + i] = 1.0f / (1.0f + expf(-lt_load(a, a_dtype, row + g_off + i)));
  if (pool == nullptr) return;                      // a layer that reads another layer's rows
  // the key/value latent and the shared rotated key part, into the token's row of the cache
  ss = 0.0f;
  for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
    const float v = lt_load(a, a_dtype, row + kv_off + i);
    ss += v * v;
  }
  ss = block_sum(ss, red);
  inv = 1.0f / sqrtf(ss / (float)kv_rank + eps);
  const int pos = __ldcg(tok_pos + t);
  const int pg = __ldcg(block_table + (int64_t)__ldcg(tok_seq + t) * bt_stride + pos / page);
  if (pg < 0) return;
  const int64_t dst = ((int64_t)pg * page + pos % page) * kv_row;
  for (int i = threadIdx.x; i < rank_pad; i += blockDim.x) {
    const float v = i < kv_rank ? lt_load(a, a_dtype, row + kv_off + i) * inv * lt_load_w(wkv, wkv_dtype, i) : 0.0f;
    lt_store(pool, pool_dtype, dst + i, v);
  }
  const int half = rot / 2;
  const int64_t src = row + kv_off + kv_rank;
  for (int i = threadIdx.x; i < kv_row - rank_pad; i += blockDim.x) {
    float v = 0.0f;
    if (i < rot) {
      const int f = i < half ? i : i - half;
      float sn, cs;
      rope_sincos((float)pos, inv_freq[f], inv_freq_lo ? inv_freq_lo[f] : 0.0f, &sn, &cs);
      const float lo = lt_load(a, a_dtype, src + f), hi = lt_load(a, a_dtype, src + f + half);
      v = i < half ? lo * cs - hi * sn : hi * cs + lo * sn;
    } else if (i < rot_dim) {
      v = lt_load(a, a_dtype, src + i);
    }
    lt_store(pool, pool_dtype, dst + rank_pad + i, v);
  }
}

// A value that an earlier kernel of the step wrote: through L2 (see load_vec_cg in common.cuh).
__device__ inline float lt_act(const float* p) { return __ldcg(p); }
__device__ inline float lt_act(const __nv_bfloat16* p) { return __bfloat162float(__ldcg(p)); }

constexpr int HG_TM = 8;          // tokens per block
constexpr int HG_TN = 32;         // outputs per block: a warp's lanes
constexpr int HG_KG = 8;          // warps of a block; each takes every eighth slice of a staged piece of K
// HG_KC, features of x staged at a time, is a parameter of the kernel: 512 for a single block of tokens (HG_KC / 8 = 64
// loads of w in flight a thread, 128 registers: two blocks an SM, which is plenty for the (N / 32) * heads blocks of a
// token's step), 128 for many tokens (16 loads, small blocks, eight of them an SM).

// A block takes 8 tokens x 32 outputs of one head.  Its eight warps split the features k between them (a warp's
// lanes read 32 consecutive outputs of one row of w: one 64- or 128-byte piece), so a token's step, which has one
// block of tokens, still has (N / 32) * heads blocks of 256 threads with K / 8 loads each in flight, and the
// partial sums meet in shared memory in the order of the warps.
template <typename T, int HG_KC>
__global__ void __launch_bounds__(HG_TN * HG_KG)
head_gemm_kernel(const T* x, int64_t x_row, int x_head, const T* __restrict__ w, T* out, int64_t out_row, int out_head,
                 int Tn, int heads, int K, int N, const float* mul, int rot_dim, int rot,
                 const float* __restrict__ inv_freq, const float* __restrict__ inv_freq_lo,
                 const int* __restrict__ tok_pos, int tail_off, int n_blocks) {
  constexpr int HG_PER = HG_KC / HG_KG;
  __shared__ float xs[HG_TM][HG_KC];
  __shared__ float part[HG_KG][HG_TM][HG_TN];
  pdl_trigger();
  const int h = blockIdx.z, t0 = blockIdx.y * HG_TM;
  if ((int)blockIdx.x >= n_blocks) {
    pdl_wait();
    // the tail of each head's output row: zeros, the rotated features, zeros
    const int half = rot / 2;
    const int span = out_head - N;
    for (int idx = threadIdx.x; idx < HG_TM * span; idx += blockDim.x) {
      const int m = idx / span, i = N + (idx - m * span), t = t0 + m;
      if (t >= Tn) continue;
      const int r = i - tail_off;
      float v = 0.0f;
      if (r >= 0 && r < rot_dim) {
        const T* src = x + (int64_t)t * x_row + (int64_t)h * x_head + K;
        if (r < rot) {
          const int f = r < half ? r : r - half;
          float sn, cs;
          rope_sincos((float)__ldcg(tok_pos + t), inv_freq[f], inv_freq_lo ? inv_freq_lo[f] : 0.0f, &sn, &cs);
          const float lo = lt_act(src + f), hi = lt_act(src + f + half);
          v = r < half ? lo * cs - hi * sn : hi * cs + lo * sn;
        } else {
          v = lt_act(src + r);
        }
      }
      Elem<T>::store(out + (int64_t)t * out_row + (int64_t)h * out_head + i, v);
    }
    return;
  }
  const int lane = threadIdx.x & 31, kg = threadIdx.x >> 5;
  const int n = blockIdx.x * HG_TN + lane;
  float acc[HG_TM];
#pragma unroll
  for (int m = 0; m < HG_TM; ++m) acc[m] = 0.0f;
  const T* wh = w + (int64_t)h * K * N;
  for (int k0 = 0; k0 < K; k0 += HG_KC) {
    const int kc = min(HG_KC, K - k0);
    // this warp's features of the piece are kg, kg + 8, ...: all their weights are asked for at once (they depend on
    // no kernel of the step, so the first piece's are on their way before the wait for the kernel before this one)
    float wv[HG_PER];
#pragma unroll
    for (int u = 0; u < HG_PER; ++u) {
      const int k = kg + u * HG_KG;
      wv[u] = (n < N && k < kc) ? Elem<T>::load(wh + (int64_t)(k0 + k) * N + n) : 0.0f;
    }
    if (k0 == 0) pdl_wait();
    __syncthreads();
    for (int idx = threadIdx.x; idx < HG_TM * HG_KC; idx += blockDim.x) {
      const int m = idx / HG_KC, k = idx - m * HG_KC, t = t0 + m;
      xs[m][k] = (t < Tn && k < kc) ? lt_act(x + (int64_t)t * x_row + (int64_t)h * x_head + k0 + k) : 0.0f;
    }
    __syncthreads();
#pragma unroll
    for (int u0 = 0; u0 < HG_PER; u0 += 16) {
      if (u0 * HG_KG < kc) {
#pragma unroll
        for (int u = u0; u < u0 + 16; ++u)
#pragma unroll
          for (int m = 0; m < HG_TM; ++m) acc[m] = fmaf(xs[m][kg + u * HG_KG], wv[u], acc[m]);
      }
    }
  }
#pragma unroll
  for (int m = 0; m < HG_TM; ++m) part[kg][m][lane] = acc[m];
  __syncthreads();
  {
    const int m = kg, t = t0 + m;                      // warp m adds up token m's partial sums, in the order of the warps
    if (n < N && t < Tn) {
      float sum = 0.0f;
#pragma unroll
      for (int g = 0; g < HG_KG; ++g) sum += part[g][m][lane];
      const float f = mul ? __ldcg(mul + (int64_t)t * heads + h) : 1.0f;
      Elem<T>::store(out + (int64_t)t * out_row + (int64_t)h * out_head + n, sum * f);
    }
  }
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_latent_prep(const void* a, int a_dtype, int lda, int T, int q_off, int q_rank, const void* wq,
                                int wq_dtype, int kv_off, int kv_rank, int rot_dim, const void* wkv, int wkv_dtype,
                                int g_off, int heads, float eps, const float* inv_freq, const float* inv_freq_lo, int rot,
                                const int* tok_pos, const int* tok_seq, const int* block_table, int bt_stride, int page,
                                void* pool, int pool_dtype, int kv_row, int rank_pad, void* cq, int cq_dtype, float* gate,
                                cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || q_rank < 1 || heads < 1 || lda < 1 || rot < 0 || rot % 2 != 0 || rot > rot_dim ||
      (pool != nullptr && (kv_rank < 1 || rot_dim < 0 || rank_pad < kv_rank || kv_row < rank_pad + rot_dim || page < 1 ||
                           (rot > 0 && inv_freq == nullptr)))) {
    set_error("latent_prep: bad sizes T=%d q_rank=%d kv_rank=%d rot_dim=%d rot=%d heads=%d row=%d rank_pad=%d", T, q_rank,
              kv_rank, rot_dim, rot, heads, kv_row, rank_pad);
    return ERR_BAD_ARGUMENT;
  }
  launch_pdl(latent_prep_kernel, dim3(T), dim3(128), 0, stream, a, a_dtype, lda, q_off, q_rank, wq, wq_dtype, kv_off,
             kv_rank, rot_dim, wkv, wkv_dtype, g_off, heads, eps, inv_freq, inv_freq_lo, rot, tok_pos, tok_seq, block_table,
             bt_stride, page, pool, pool_dtype, kv_row, rank_pad, cq, cq_dtype, gate);
  return launch_status("latent_prep");
}

extern "C" int exl3_head_gemm(const void* x, int64_t x_row, int x_head, const void* w, void* out, int64_t out_row,
                              int out_head, int dtype, int T, int heads, int K, int N, const float* mul, int rot_dim,
                              int rot, const float* inv_freq, const float* inv_freq_lo, const int* tok_pos, int tail_off,
                              cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || heads < 1 || heads > 65535 || K < 1 || N < 1 || out_head < N || rot_dim < 0 || rot < 0 || rot % 2 != 0 ||
      rot > rot_dim || (rot_dim > 0 && (tail_off < N || tail_off + rot_dim > out_head || tok_pos == nullptr ||
                                        (rot > 0 && inv_freq == nullptr)))) {
    set_error("head_gemm: bad sizes T=%d heads=%d K=%d N=%d out_head=%d rot_dim=%d rot=%d tail=%d", T, heads, K, N,
              out_head, rot_dim, rot, tail_off);
    return ERR_BAD_ARGUMENT;
  }
  const int n_blocks = w == nullptr ? 0 : ceil_div(N, HG_TN);     // no weights: only the tails are written
  const int tail = out_head > N ? 1 : 0;
  const int rows = ceil_div(T, HG_TM);
  if (n_blocks + tail == 0) return 0;
  if (rows > 65535) {
    // grid.y is limited: walk the tokens in slabs
    const int slab = 65535 * HG_TM;
    for (int t0 = 0; t0 < T; t0 += slab) {
      const int n = T - t0 < slab ? T - t0 : slab;
      const size_t es = dtype == DT_F32 ? 4 : 2;
      int rc = exl3_head_gemm(static_cast<const char*>(x) + (size_t)t0 * x_row * es, x_row, x_head, w,
                              static_cast<char*>(out) + (size_t)t0 * out_row * es, out_row, out_head, dtype, n, heads, K,
                              N, mul ? mul + (size_t)t0 * heads : nullptr, rot_dim, rot, inv_freq, inv_freq_lo,
                              tok_pos ? tok_pos + t0 : nullptr, tail_off, stream);
      if (rc) return rc;
    }
    return 0;
  }
  dim3 grid(n_blocks + tail, rows, heads);
#define EXL3_HG(TT, KC)                                                                                              \
  launch_pdl(head_gemm_kernel<TT, KC>, grid, dim3(HG_TN * HG_KG), 0, stream, static_cast<const TT*>(x), x_row, x_head,  \
             static_cast<const TT*>(w), static_cast<TT*>(out), out_row, out_head, T, heads, K, N, mul, rot_dim, rot,    \
             inv_freq, inv_freq_lo, tok_pos, tail_off, n_blocks)
  const bool few = rows == 1 && K > 128;
  if (dtype == DT_F32) {
    if (few) EXL3_HG(float, 512); else EXL3_HG(float, 128);
  } else if (dtype == DT_BF16) {
    if (few) EXL3_HG(__nv_bfloat16, 512); else EXL3_HG(__nv_bfloat16, 128);
  } else {
    set_error("head_gemm: unsupported element type %d", dtype);
    return ERR_UNSUPPORTED;
  }
#undef EXL3_HG
  return launch_status("head_gemm");
}
