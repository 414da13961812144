// What lies between an attention's joint input projection and the attention itself, in one kernel:
//
//   queries and keys, head by head: x <- x / sqrt(mean(x^2) + eps) (* w)         (norm 1 / 2; 0: as they are)
//   rotary encoding of the first `rot` features at the token's position p, angle a_i = p f_i:
//       layout 0 pairs feature i with i + rot / 2, layout 1 feature 2i with 2i + 1;
//       (u, v) <- (u cos a - v sin a, v cos a + u sin a), sines and cosines times mscale
//   keys times k_mul
//   values: v <- (1 - lambda) v + lambda v_src   when a mixing weight is given (v_src: another layer's values of
//       the same token)
//   queries to q_out; keys and values to the token's place in the paged cache, or keys to k_out when there is no
//   cache (mixers that keep a state instead).
//
// Rows of q_out, k_out and the cache hold hd_pad >= hd (hdv_pad >= hdv) features; the features beyond a head's own
// are written as zeros, so that kernels which read rows in 16-byte pieces take any even head size.  All arithmetic
// is float32; inputs and outputs have their own element types.
#include "api.h"
#include "common.cuh"

namespace exl3 {

__device__ inline float qp_load(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? static_cast<const float*>(p)[i]
                         : __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ inline float qp_load_act(const void* p, int dtype, int64_t i) {
  return dtype == DT_F32 ? __ldcg(static_cast<const float*>(p) + i)
                         : __bfloat162float(__ldcg(static_cast<const __nv_bfloat16*>(p) + i));
}
__device__ inline void qp_store(void* p, int dtype, int64_t i, float v) {
  if (dtype == DT_F32) static_cast<float*>(p)[i] = v;
  else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

constexpr int QP_WARPS = 8;
constexpr int QP_TABLE = 128;                    // pairs whose sine and cosine a block works out once for its token

struct QkPrepArgs {
  const void* x; int x_dtype; int64_t ld; int q_off, k_off, v_off;
  int nh, nkv, hd, hdv, hd_pad, hdv_pad;
  int norm; const void* q_w; const void* k_w; int w_dtype; float eps;
  int rot, layout; const float* f_hi; const float* f_lo; float mscale, k_mul;
  const void* lambda; int lambda_dtype; const void* v_src; int v_src_dtype; int64_t v_src_ld;
  const int* tok_pos; const int* tok_seq; const int* block_table; int bt_stride, page;
  void* q_out; int q_out_dtype; void* k_out; int k_out_dtype; void* k_pool; void* v_pool; int pool_dtype;
};

// Block (t, y) takes the heads y * per_block .. of token t, a warp a head at a time.  A head a warp (per_block =
// QP_WARPS) is what the entry point asks for: a warp that walks several heads in turn waits for each one's loads
// (2,048 tokens with 48 heads of 128: 61 us with twelve heads a warp).
__global__ void __launch_bounds__(QP_WARPS * 32) qk_prep_kernel(QkPrepArgs a, int per_block) {
  extern __shared__ float qp_sm[];                    // [QP_WARPS][max(hd, hdv)]
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int wide = max(a.hd, a.hdv);
  float* sm = qp_sm + warp * wide;
  const int pos = __ldcg(a.tok_pos + t);
  int pg = -1;
  if (a.k_pool != nullptr)
    pg = __ldcg(a.block_table + (int64_t)__ldcg(a.tok_seq + t) * a.bt_stride + pos / a.page);
  const int in_page = a.k_pool != nullptr ? pos % a.page : 0;
  const int jobs = a.nh + a.nkv + (a.v_off >= 0 ? a.nkv : 0);
  const float fpos = (float)pos;
  // the token's sines and cosines (times mscale), once for all its heads
  __shared__ float s_sn[QP_TABLE], s_cs[QP_TABLE];
  const int half = a.rot >> 1;
  const bool table = half <= QP_TABLE;
  if (table) {
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      float sn, cs;
      rope_sincos(fpos, a.f_hi[i], a.f_lo ? a.f_lo[i] : 0.0f, &sn, &cs);
      s_sn[i] = sn * a.mscale;
      s_cs[i] = cs * a.mscale;
    }
    __syncthreads();
  }
  const int job_end = min(jobs, ((int)blockIdx.y + 1) * per_block);
  for (int job = (int)blockIdx.y * per_block + warp; job < job_end; job += QP_WARPS) {
    const bool is_q = job < a.nh;
    const bool is_k = !is_q && job < a.nh + a.nkv;
    const int head = is_q ? job : (is_k ? job - a.nh : job - a.nh - a.nkv);
    if (!is_q && !is_k) {
      // a value head
      const int64_t src = (int64_t)t * a.ld + a.v_off + (int64_t)head * a.hdv;
      float lam = 0.0f;
      if (a.lambda != nullptr) lam = qp_load(a.lambda, a.lambda_dtype, 0);
      if (a.v_pool == nullptr || pg < 0) continue;
      const int64_t dst = (((int64_t)pg * a.nkv + head) * a.page + in_page) * a.hdv_pad;
      for (int e = lane; e < a.hdv_pad; e += 32) {
        float v = 0.0f;
        if (e < a.hdv) {
          v = qp_load_act(a.x, a.x_dtype, src + e);
          if (a.lambda != nullptr) {
            const float o = qp_load_act(a.v_src, a.v_src_dtype, (int64_t)t * a.v_src_ld + (int64_t)head * a.hdv + e);
            v = (1.0f - lam) * v + lam * o;
          }
        }
        qp_store(a.v_pool, a.pool_dtype, dst + e, v);
      }
      continue;
    }
    const int64_t src = (int64_t)t * a.ld + (is_q ? a.q_off : a.k_off) + (int64_t)head * a.hd;
    float ss = 0.0f;
    for (int e = lane; e < a.hd; e += 32) {
      const float v = qp_load_act(a.x, a.x_dtype, src + e);
      sm[e] = v;
      ss += v * v;
    }
    float inv = 1.0f;
    if (a.norm) {
      ss = warp_sum(ss);
      inv = 1.0f / sqrtf(ss / (float)a.hd + a.eps);
    }
    __syncwarp();
    const void* w = a.norm == 2 ? (is_q ? a.q_w : a.k_w) : nullptr;
    const float mul = is_k ? a.k_mul : 1.0f;
    void* out;
    int out_dtype;
    int64_t dst;
    if (is_q) {
      out = a.q_out; out_dtype = a.q_out_dtype;
      dst = ((int64_t)t * a.nh + head) * a.hd_pad;
    } else if (a.k_pool != nullptr) {
      if (pg < 0) { __syncwarp(); continue; }
      out = a.k_pool; out_dtype = a.pool_dtype;
      dst = (((int64_t)pg * a.nkv + head) * a.page + in_page) * a.hd_pad;
    } else {
      out = a.k_out; out_dtype = a.k_out_dtype;
      dst = ((int64_t)t * a.nkv + head) * a.hd_pad;
    }
    for (int e = lane; e < a.hd_pad; e += 32) {
      float v = 0.0f;
      if (e < a.hd) {
        v = sm[e] * inv * (w ? qp_load(w, a.w_dtype, e) : 1.0f);
        if (e < a.rot) {
          int i, pe;
          bool second;
          if (a.layout == 1) { i = e >> 1; second = e & 1; pe = e ^ 1; }
          else { second = e >= half; i = second ? e - half : e; pe = second ? e - half : e + half; }
          const float o = sm[pe] * inv * (w ? qp_load(w, a.w_dtype, pe) : 1.0f);
          float sn, cs;
          if (table) {
            sn = s_sn[i];
            cs = s_cs[i];
          } else {
            rope_sincos(fpos, a.f_hi[i], a.f_lo ? a.f_lo[i] : 0.0f, &sn, &cs);
            sn *= a.mscale;
            cs *= a.mscale;
          }
          v = second ? fmaf(v, cs, o * sn) : fmaf(v, cs, -o * sn);
        }
        v *= mul;
      }
      qp_store(out, out_dtype, dst + e, v);
    }
    __syncwarp();                                       // the warp's row of shared memory is free again
  }
}

// The common case with 16-byte accesses: bfloat16 queries and cache, head sizes in multiples of 8 (no padding), pairs
// of neighbouring features rotated (layout 1) or none, so that a pair lies inside the eight features that a lane holds.
// A head takes LPH = 2, 4, ... 32 lanes (the power of two that covers hd / 8 and hdv / 8), so a warp works on 32 / LPH
// heads side by side; block (t, y) takes the heads y * QP_WARPS * (32 / LPH) ... of token t.
template <typename TX>
__device__ inline void qp_load8(const TX* p, float (&v)[8]);
template <>
__device__ inline void qp_load8<float>(const float* p, float (&v)[8]) {
  float a[4], b[4];
  load_vec_cg(p, a);
  load_vec_cg(p + 4, b);
#pragma unroll
  for (int e = 0; e < 4; ++e) { v[e] = a[e]; v[4 + e] = b[e]; }
}
template <>
__device__ inline void qp_load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&v)[8]) { load_vec_cg(p, v); }

template <typename TX, typename TS>
__global__ void __launch_bounds__(QP_WARPS * 32) qk_prep_vec_kernel(QkPrepArgs a, int lph) {
  __shared__ float s_sn[QP_TABLE], s_cs[QP_TABLE];
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int pos = __ldcg(a.tok_pos + t);
  const int pg = __ldcg(a.block_table + (int64_t)__ldcg(a.tok_seq + t) * a.bt_stride + pos / a.page);
  const int in_page = pos % a.page;
  const int half = a.rot >> 1;
  for (int i = threadIdx.x; i < half; i += blockDim.x) {
    float sn, cs;
    rope_sincos((float)pos, a.f_hi[i], a.f_lo ? a.f_lo[i] : 0.0f, &sn, &cs);
    s_sn[i] = sn * a.mscale;
    s_cs[i] = cs * a.mscale;
  }
  __syncthreads();
  const int per_warp = 32 / lph;
  const int jobs = a.nh + 2 * a.nkv;
  const int job = ((int)blockIdx.y * QP_WARPS + warp) * per_warp + lane / lph;
  const int e0 = (lane % lph) * 8;
  const bool live = job < jobs;
  const bool is_q = job < a.nh, is_k = !is_q && job < a.nh + a.nkv;
  const int head = is_q ? job : (is_k ? job - a.nh : job - a.nh - a.nkv);
  const TX* x = static_cast<const TX*>(a.x) + (int64_t)t * a.ld;
  __nv_bfloat16* kp = static_cast<__nv_bfloat16*>(a.k_pool);
  __nv_bfloat16* vp = static_cast<__nv_bfloat16*>(a.v_pool);
  float v[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) v[e] = 0.0f;
  if (live && !is_q && !is_k) {
    // a value head
    if (e0 < a.hdv && pg >= 0) {
      qp_load8<TX>(x + a.v_off + (int64_t)head * a.hdv + e0, v);
      if (a.lambda != nullptr) {
        const float lam = qp_load(a.lambda, a.lambda_dtype, 0);
        float o[8];
        qp_load8<TS>(static_cast<const TS*>(a.v_src) + (int64_t)t * a.v_src_ld + (int64_t)head * a.hdv + e0, o);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = (1.0f - lam) * v[e] + lam * o[e];
      }
      store_vec(vp + (((int64_t)pg * a.nkv + head) * a.page + in_page) * a.hdv + e0, v);
    }
  }
  const bool qk = live && (is_q || is_k);
  const bool mine = qk && e0 < a.hd;
  if (mine) qp_load8<TX>(x + (is_q ? a.q_off : a.k_off) + (int64_t)head * a.hd + e0, v);
  float inv = 1.0f;
  if (a.norm) {
    // every lane takes part in the shuffles; a head's lanes are neighbours
    float ss = 0.0f;
    if (mine) {
#pragma unroll
      for (int e = 0; e < 8; ++e) ss += v[e] * v[e];
    }
    for (int o = lph >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    inv = 1.0f / sqrtf(ss / (float)a.hd + a.eps);
  }
  if (!mine) return;
  if (a.norm == 2) {
    float w[8];
    const float* wp = static_cast<const float*>(is_q ? a.q_w : a.k_w) + e0;
    load_vec(wp, reinterpret_cast<float(&)[4]>(w[0]));
    load_vec(wp + 4, reinterpret_cast<float(&)[4]>(w[4]));
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] *= inv * w[e];
  } else {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] *= inv;
  }
  if (e0 < a.rot) {                                    // rot is a multiple of 8 here: all of the lane's pairs or none
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const float sn = s_sn[(e0 >> 1) + p], cs = s_cs[(e0 >> 1) + p];
      const float u = v[2 * p], w2 = v[2 * p + 1];
      v[2 * p] = fmaf(u, cs, -w2 * sn);
      v[2 * p + 1] = fmaf(w2, cs, u * sn);
    }
  }
  if (is_q) {
    store_vec(static_cast<__nv_bfloat16*>(a.q_out) + ((int64_t)t * a.nh + head) * a.hd + e0, v);
  } else if (pg >= 0) {
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] *= a.k_mul;
    store_vec(kp + (((int64_t)pg * a.nkv + head) * a.page + in_page) * a.hd + e0, v);
  }
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_qk_prep(const void* x, int x_dtype, int64_t ld, int q_off, int k_off, int v_off, int T, int nh,
                            int nkv, int hd, int hdv, int hd_pad, int hdv_pad, int norm, const void* q_w,
                            const void* k_w, int w_dtype, float eps, int rot, int layout, const float* inv_freq,
                            const float* inv_freq_lo, float mscale, float k_mul, const void* mix_lambda,
                            int lambda_dtype, const void* v_src, int v_src_dtype, int64_t v_src_ld, const int* tok_pos,
                            const int* tok_seq, const int* block_table, int bt_stride, int page, void* q_out,
                            int q_out_dtype, void* k_out, int k_out_dtype, void* k_pool, void* v_pool, int pool_dtype,
                            cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || nh < 1 || nkv < 1 || hd < 1 || hd_pad < hd || (v_off >= 0 && (hdv < 1 || hdv_pad < hdv)) ||
      norm < 0 || norm > 2 || rot < 0 || rot > hd || rot % 2 != 0 || layout < 0 || layout > 1 ||
      (rot > 0 && inv_freq == nullptr) || (norm == 2 && (q_w == nullptr || k_w == nullptr)) || q_out == nullptr ||
      (k_pool == nullptr && k_out == nullptr) || (k_pool != nullptr && (block_table == nullptr || page < 1)) ||
      (v_off >= 0 && k_pool != nullptr && v_pool == nullptr) || (mix_lambda != nullptr && v_src == nullptr)) {
    set_error("qk_prep: bad arguments T=%d heads=%d/%d head_dim=%d (%d) value_dim=%d (%d) norm=%d rot=%d layout=%d",
              T, nh, nkv, hd, hd_pad, hdv, hdv_pad, norm, rot, layout);
    return ERR_BAD_ARGUMENT;
  }
  QkPrepArgs a;
  a.x = x; a.x_dtype = x_dtype; a.ld = ld; a.q_off = q_off; a.k_off = k_off; a.v_off = v_off;
  a.nh = nh; a.nkv = nkv; a.hd = hd; a.hdv = v_off >= 0 ? hdv : 0; a.hd_pad = hd_pad; a.hdv_pad = hdv_pad;
  a.norm = norm; a.q_w = q_w; a.k_w = k_w; a.w_dtype = w_dtype; a.eps = eps;
  a.rot = rot; a.layout = layout; a.f_hi = inv_freq; a.f_lo = inv_freq_lo; a.mscale = mscale; a.k_mul = k_mul;
  a.lambda = mix_lambda; a.lambda_dtype = lambda_dtype; a.v_src = v_src; a.v_src_dtype = v_src_dtype;
  a.v_src_ld = v_src_ld;
  a.tok_pos = tok_pos; a.tok_seq = tok_seq; a.block_table = block_table; a.bt_stride = bt_stride; a.page = page;
  a.q_out = q_out; a.q_out_dtype = q_out_dtype; a.k_out = k_out; a.k_out_dtype = k_out_dtype;
  a.k_pool = k_pool; a.v_pool = v_pool; a.pool_dtype = pool_dtype;
  // the common case with 16-byte accesses (see qk_prep_vec_kernel)
  const int widest = hd > a.hdv ? hd : a.hdv;
  const bool src_ok = mix_lambda == nullptr || ((v_src_dtype == DT_BF16 || v_src_dtype == DT_F32) && v_src_ld % 8 == 0 &&
                                                aligned16(v_src));
  if (k_pool != nullptr && v_off >= 0 && pool_dtype == DT_BF16 && q_out_dtype == DT_BF16 && hd % 8 == 0 && hdv % 8 == 0 &&
      hd_pad == hd && hdv_pad == hdv && widest <= 256 && ld % 8 == 0 && q_off % 8 == 0 && k_off % 8 == 0 &&
      v_off % 8 == 0 && (rot == 0 || (layout == 1 && rot % 8 == 0 && rot / 2 <= QP_TABLE)) &&
      (norm != 2 || w_dtype == DT_F32) && (x_dtype == DT_BF16 || x_dtype == DT_F32) && aligned16(x) && aligned16(q_out) &&
      aligned16(k_pool) && aligned16(v_pool) && src_ok && (norm != 2 || (aligned16(q_w) && aligned16(k_w)))) {
    int lph = 1;
    while (lph * 8 < widest) lph <<= 1;
    const int per_block = QP_WARPS * (32 / lph);
    const int jobs = nh + 2 * nkv;
    const dim3 grid(T, ceil_div(jobs, per_block)), threads(QP_WARPS * 32);
    const bool xf = x_dtype == DT_F32, sf = mix_lambda != nullptr && v_src_dtype == DT_F32;
    if (xf && sf) launch_pdl(qk_prep_vec_kernel<float, float>, grid, threads, 0, stream, a, lph);
    else if (xf) launch_pdl(qk_prep_vec_kernel<float, __nv_bfloat16>, grid, threads, 0, stream, a, lph);
    else if (sf) launch_pdl(qk_prep_vec_kernel<__nv_bfloat16, float>, grid, threads, 0, stream, a, lph);
    else launch_pdl(qk_prep_vec_kernel<__nv_bfloat16, __nv_bfloat16>, grid, threads, 0, stream, a, lph);
    return launch_status("qk_prep");
  }
  const size_t smem = (size_t)QP_WARPS * (hd > a.hdv ? hd : a.hdv) * sizeof(float);
  if (smem > 48 * 1024) { set_error("qk_prep: heads of %d features are too wide", hd); return ERR_UNSUPPORTED; }
  const int jobs = nh + nkv + (v_off >= 0 ? nkv : 0);
  const int per_block = QP_WARPS;
  const int groups = ceil_div(jobs, per_block);
  if (groups > 65535) { set_error("qk_prep: too many heads"); return ERR_UNSUPPORTED; }
  launch_pdl(qk_prep_kernel, dim3(T, groups), dim3(QP_WARPS * 32), smem, stream, a, per_block);
  return launch_status("qk_prep");
}
