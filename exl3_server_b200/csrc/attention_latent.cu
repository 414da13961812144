// Attention over latent rows on the tensor cores (bfloat16): every head of a token reads the same cached row
// [ c (values, dv features) | rotated key part | padding ] of dk features, so the query rows of one sequence,
// flattened over (token, head), are ONE matrix Q [rows, dk] against ONE key matrix K [keys, dk] whose leading dv
// columns are also the values:
//
//   S = Q K^T * scale,  row f = (token f / H, head f % H) sees keys j <= pos0 + f / H,  O = softmax(S) K[:, :dv]
//
// One kernel serves prompts, portions of prompts and single tokens.  A block of eight warps takes a tile of
// 16 * MT consecutive rows of one sequence and walks the sequence's pages (64 keys, one page a step, the next page
// on its way by cp.async while this one is worked on).  All warps share all rows: for the scores a warp owns 8 of
// the page's 64 keys (its B fragments serve every row tile), for the output it owns every eighth 16-column slice
// of the values (its B fragments, read transposed out of the very tile the keys came from, again serve every row
// tile).  Row maxima and sums meet in shared memory; the running maximum, the running sum and the output
// accumulators are float32, the probabilities are rounded to bfloat16 for the second product.  With n_splits > 1 a
// block takes only the pages of one chunk (chunks are aligned to absolute positions) and leaves a record
// [dv sums, maximum, sum] per row and chunk, which latent_combine_kernel merges in chunk order.
//
// Two forms.  Tiles of three or four sixteens of rows (prompts): the eight warps issue the next page's 16-byte copies
// themselves.  Tiles of one or two (decoded tokens): four more warps do nothing but copy; they and the eight others
// hand the two key buffers back and forth through named barriers (2 + buffer: the page has landed; 4 + buffer: the
// buffer is free again), every one of which each thread of the block reaches the same number of times.
//
// Exponentials are base 2: scores carry scale * log2(e), maxima are in those units everywhere.
#include "api.h"
#include "common.cuh"

#include <math.h>
#include <stdlib.h>

namespace exl3 {

constexpr int LA_WARPS = 8;
constexpr int LA_THREADS = LA_WARPS * 32;
constexpr int LA_KEYS = 64;                // keys per step: one page
constexpr int LA_PAD = 8;                  // elements added to a shared-memory row: 16-byte pieces of consecutive rows fall into different banks
constexpr int LA_COPY_WARPS = 4;           // warps that only copy pages, in the kernel's form that has them
constexpr int LA_MAX_PAIRS = 4;            // 16-column slices of the values per warp: dv <= 8 * 4 * 16 = 512

__device__ inline void la_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ inline void la_ldmatrix_x2(uint32_t (&r)[2], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ inline void la_ldmatrix_x4_trans(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ inline void la_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ inline void la_cp_async16(void* dst, const void* src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ inline void la_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ inline void la_cp_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }
__device__ inline void la_bar_sync(int id, int count) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ inline void la_bar_arrive(int id, int count) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(count) : "memory"); }
__device__ inline float la_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// PW: four more warps do nothing but copy the pages (see the top of the file); the eight others then meet at named
// barriers: 1 among themselves, 2 + buffer when a page has landed, 4 + buffer when they are done with it.
template <int MT, bool PW>
__global__ void __launch_bounds__(LA_THREADS + (PW ? 32 * LA_COPY_WARPS : 0), 1)
attn_latent_kernel(const __nv_bfloat16* q, __nv_bfloat16* out, const __nv_bfloat16* pool, const int* __restrict__ block_table,
                   int bt_stride, const int* __restrict__ row_start, const int* __restrict__ row_pos0, int H, int dk, int dv,
                   float scale_log2, int pages_per_chunk, int n_splits, float* scratch, const float* gate) {
  constexpr int M = 16 * MT;
  extern __shared__ __align__(16) unsigned char la_smem[];
  const int ldk = dk + LA_PAD;                      // elements per shared-memory row of Q and K
  constexpr int ldp = LA_KEYS + LA_PAD;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(la_smem);
  __nv_bfloat16* Ks = Qs + (size_t)M * ldk;         // two tiles of LA_KEYS rows
  __nv_bfloat16* Ps = Ks + (size_t)2 * LA_KEYS * ldk;
  float* red_max = reinterpret_cast<float*>(Ps + (size_t)M * ldp);   // [LA_WARPS][M]
  float* red_sum = red_max + LA_WARPS * M;          // [LA_WARPS][M]
  float* m_run = red_sum + LA_WARPS * M;            // [M]
  float* l_run = m_run + M;                         // [M]
  float* corr = l_run + M;                          // [M]

  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.y, sp = blockIdx.z;                 // tiles along x: a long prompt of many heads has many
  const int tok0 = __ldcg(row_start + b);
  const int F = (__ldcg(row_start + b + 1) - tok0) * H;      // rows of this sequence in this step
  const int f0 = blockIdx.x * M;
  if (f0 >= F) return;
  const int pos0 = __ldcg(row_pos0 + b);
  const int rows = min(M, F - f0);
  const int last_pos = pos0 + (f0 + rows - 1) / H;           // the tile's last row sees keys up to here
  int page_lo = 0, page_hi = last_pos / LA_KEYS;             // inclusive
  if (n_splits > 1) {
    page_lo = sp * pages_per_chunk;
    page_hi = min(page_hi, page_lo + pages_per_chunk - 1);
  }
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int* bt = block_table + (int64_t)b * bt_stride;
  const int vecs = dk / 8;                                   // 16-byte pieces per row

  constexpr int ALL = LA_THREADS + 32 * LA_COPY_WARPS;              // the threads that meet at the barriers between the copying warp and the others
  auto sync_compute = [&]() {
    if constexpr (PW) la_bar_sync(1, LA_THREADS); else __syncthreads();
  };
  // a thread's pieces of a key tile: piece i = index + copiers * n lies in row r(n), column c(n), stepped without dividing
  constexpr int COPIERS = PW ? 32 * LA_COPY_WARPS : LA_THREADS;
  const int ci = PW ? tid - LA_THREADS : tid;         // (meaningful in the copying warps only when there are such)
  const int step_r = COPIERS / vecs, step_c = COPIERS % vecs;
  const int first_r = ci / vecs, first_c = ci % vecs;
  auto load_keys = [&](int pg, int buf) {
    __nv_bfloat16* dst = Ks + (size_t)buf * LA_KEYS * ldk;
    int r = first_r, c = first_c;
    while (r < LA_KEYS) {
      if (pg >= 0) la_cp_async16(dst + (size_t)r * ldk + c * 8, pool + ((int64_t)pg * LA_KEYS + r) * dk + c * 8);
      else *reinterpret_cast<uint4*>(dst + (size_t)r * ldk + c * 8) = make_uint4(0, 0, 0, 0);
      r += step_r;
      c += step_c;
      if (c >= vecs) { c -= vecs; ++r; }
    }
  };
  // page numbers are fetched one step before the copy that needs them, so that no copy waits for its address
  int pg_next = page_lo <= page_hi ? __ldcg(bt + page_lo) : -1;
  if constexpr (PW) {
    if (warp >= LA_WARPS) {
      // the copying warp: a page into the buffer that the others have let go of, then the word that it has landed
      for (int pi = page_lo; pi <= page_hi; ++pi) {
        const int buf = (pi - page_lo) & 1;
        const int pg = pg_next;
        pg_next = pi + 1 <= page_hi ? __ldcg(bt + pi + 1) : -1;
        if (pi - page_lo >= 2) la_bar_sync(4 + buf, ALL);
        load_keys(pg, buf);
        la_cp_commit();
        la_cp_wait_all();
        __threadfence_block();
        la_bar_arrive(2 + buf, ALL);
      }
      return;
    }
  } else {
    if (page_lo <= page_hi) load_keys(pg_next, 0);
    la_cp_commit();
    pg_next = page_lo + 1 <= page_hi ? __ldcg(bt + page_lo + 1) : -1;
  }
  // the queries of the tile; rows beyond the sequence's are zero
  for (int i = tid; i < M * vecs; i += LA_THREADS) {
    const int r = i / vecs, c = (i - r * vecs) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rows) v = __ldcg(reinterpret_cast<const uint4*>(q + ((int64_t)tok0 * H + f0 + r) * dk + c));
    *reinterpret_cast<uint4*>(Qs + (size_t)r * ldk + c) = v;
  }
  if (tid < M) { m_run[tid] = -INFINITY; l_run[tid] = 0.0f; }
  if constexpr (PW) sync_compute();                          // (without a copying warp the loop's first barrier does this)

  float o[MT][LA_MAX_PAIRS][2][4];
#pragma unroll
  for (int mt = 0; mt < MT; ++mt)
#pragma unroll
    for (int i = 0; i < LA_MAX_PAIRS; ++i)
#pragma unroll
      for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
        for (int e = 0; e < 4; ++e) o[mt][i][h2][e] = 0.0f;

  const int qr = lane >> 2, qc = (lane & 3) * 2;             // this lane's row and first column inside a fragment
  // ldmatrix addresses: A (x4): row lane % 16 of the row tile, column + 8 for lanes 16..31;
  // B (x2) for the scores: row lane % 8 of the warp's keys, column + 8 for lanes 8..15;
  // B (x4, transposed) for the values: key (lane % 8) + 8 * ((lane / 8) % 2), column + 8 for lanes 16..31
  const int a_row = lane & 15, a_col = (lane >> 4) * 8;
  const int bk_row = warp * 8 + (lane & 7), bk_col = ((lane >> 3) & 1) * 8;
  const int bv_row = (lane & 7) + ((lane >> 3) & 1) * 8, bv_col = (lane >> 4) * 8;

  for (int pi = page_lo; pi <= page_hi; ++pi) {
    const int buf = (pi - page_lo) & 1;
    if constexpr (PW) {
      la_bar_sync(2 + buf, ALL);                             // this page's keys have landed
    } else {
      la_cp_wait_all();
      __syncthreads();                                       // this page's keys (and, the first time, Q) are in place
      if (pi + 1 <= page_hi) load_keys(pg_next, buf ^ 1);    // that buffer's last readers passed the barrier above
      la_cp_commit();
      pg_next = pi + 2 <= page_hi ? __ldcg(bt + pi + 2) : -1;
    }
    const __nv_bfloat16* Kt = Ks + (size_t)buf * LA_KEYS * ldk;

    // scores of all rows against this warp's 8 keys
    // (with few row tiles the features go round KS sums per tile, so that the chain of dependent products is short)
    constexpr int KS = MT >= 3 ? 1 : 4 / MT;
    float sk[MT][KS][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int u = 0; u < KS; ++u) { sk[mt][u][0] = sk[mt][u][1] = sk[mt][u][2] = sk[mt][u][3] = 0.0f; }
    // (the instructions below keep their order: a group's fragments are asked for before the group before it is
    // multiplied, so that loads and products overlap)
    uint32_t bfr[2][KS][2], afr[2][KS][MT][4];
    auto load_group = [&](int k0, int which) {
#pragma unroll
      for (int u = 0; u < KS; ++u) {
        const int kk = k0 + 16 * u;
        if (kk < dk) {
          la_ldmatrix_x2(bfr[which][u], Kt + (size_t)bk_row * ldk + kk + bk_col);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) la_ldmatrix_x4(afr[which][u][mt], Qs + (size_t)(mt * 16 + a_row) * ldk + kk + a_col);
        }
      }
    };
    auto mul_group = [&](int k0, int which) {
#pragma unroll
      for (int u = 0; u < KS; ++u) {
        if (k0 + 16 * u < dk) {
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) la_mma(sk[mt][u], afr[which][u][mt], bfr[which][u][0], bfr[which][u][1]);
        }
      }
    };
    load_group(0, 0);
    for (int k0 = 0; k0 < dk; k0 += 32 * KS) {
      if (k0 + 16 * KS < dk) load_group(k0 + 16 * KS, 1);
      mul_group(k0, 0);
      if (k0 + 32 * KS < dk) load_group(k0 + 32 * KS, 0);
      if (k0 + 16 * KS < dk) mul_group(k0 + 16 * KS, 1);
    }
    float s[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float v = sk[mt][0][e];
#pragma unroll
        for (int u = 1; u < KS; ++u) v += sk[mt][u][e];
        s[mt][e] = v;
      }
    const int key0 = pi * LA_KEYS + warp * 8 + qc;           // this lane's first key (absolute position)
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = mt * 16 + qr + half * 8;
        const int lim = r < rows ? pos0 + (f0 + r) / H : -1; // keys beyond the row's own position are not seen
        float v0 = key0 <= lim ? s[mt][half * 2] * scale_log2 : -INFINITY;
        float v1 = key0 + 1 <= lim ? s[mt][half * 2 + 1] * scale_log2 : -INFINITY;
        s[mt][half * 2] = v0;
        s[mt][half * 2 + 1] = v1;
        float mx = fmaxf(v0, v1);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        if ((lane & 3) == 0) red_max[warp * M + r] = mx;
      }
    }
    sync_compute();
    if (tid < M) {
      float mx = red_max[tid];
#pragma unroll
      for (int w = 1; w < LA_WARPS; ++w) mx = fmaxf(mx, red_max[w * M + tid]);
      const float mo = m_run[tid], mn = fmaxf(mo, mx);
      corr[tid] = mn == -INFINITY ? 1.0f : la_exp2(mo - mn);      // exp2(-inf) = 0 the first time
      m_run[tid] = mn;
    }
    sync_compute();
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int r = mt * 16 + qr + half * 8;
        const float mn = m_run[r];
        const float p0 = mn == -INFINITY ? 0.0f : la_exp2(s[mt][half * 2] - mn);
        const float p1 = mn == -INFINITY ? 0.0f : la_exp2(s[mt][half * 2 + 1] - mn);
        const __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
        *reinterpret_cast<__nv_bfloat162*>(Ps + (size_t)r * ldp + warp * 8 + qc) = pb;
        // the sum takes what the second product takes: the rounded probabilities
        float sm = __bfloat162float(pb.x) + __bfloat162float(pb.y);
        sm += __shfl_xor_sync(0xffffffffu, sm, 1);
        sm += __shfl_xor_sync(0xffffffffu, sm, 2);
        if ((lane & 3) == 0) red_sum[warp * M + r] = sm;
      }
    }
    sync_compute();
    if (tid < M) {
      float sm = 0.0f;
#pragma unroll
      for (int w = 0; w < LA_WARPS; ++w) sm += red_sum[w * M + tid];
      l_run[tid] = l_run[tid] * corr[tid] + sm;
    }
    // the output: O = O * corr + P V for this warp's slices of the values
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
      const float c0 = corr[mt * 16 + qr], c1 = corr[mt * 16 + qr + 8];
#pragma unroll
      for (int i = 0; i < LA_MAX_PAIRS; ++i)
#pragma unroll
        for (int h2 = 0; h2 < 2; ++h2) {
          o[mt][i][h2][0] *= c0; o[mt][i][h2][1] *= c0;
          o[mt][i][h2][2] *= c1; o[mt][i][h2][3] *= c1;
        }
    }
#pragma unroll
    for (int kk = 0; kk < LA_KEYS; kk += 16) {
      uint32_t pf[MT][4], vf[LA_MAX_PAIRS][4];
#pragma unroll
      for (int mt = 0; mt < MT; ++mt) la_ldmatrix_x4(pf[mt], Ps + (size_t)(mt * 16 + a_row) * ldp + kk + a_col);
#pragma unroll
      for (int i = 0; i < LA_MAX_PAIRS; ++i) {
        const int col = (warp + LA_WARPS * i) * 16;
        if (col < dv) la_ldmatrix_x4_trans(vf[i], Kt + (size_t)(kk + bv_row) * ldk + col + bv_col);
      }
#pragma unroll
      for (int i = 0; i < LA_MAX_PAIRS; ++i) {
        const int col = (warp + LA_WARPS * i) * 16;
        if (col < dv) {
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            la_mma(o[mt][i][0], pf[mt], vf[i][0], vf[i][1]);
            la_mma(o[mt][i][1], pf[mt], vf[i][2], vf[i][3]);
          }
        }
      }
    }
    if constexpr (PW) {
      if (pi + 2 <= page_hi) la_bar_arrive(4 + buf, ALL);    // the copying warp may fill this buffer again
    }
    sync_compute();                                          // P, the statistics and (without a copying warp) this key tile are free again
  }
  la_cp_wait_all();
  sync_compute();                                            // the statistics, also when the chunk held no page

  // results: rows qr and qr + 8 of every row tile, this warp's column slices
#pragma unroll
  for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = mt * 16 + qr + half * 8;
      if (r >= rows) continue;
      const int64_t flat = (int64_t)tok0 * H + f0 + r;
      const float l = l_run[r], mx = m_run[r];
      if (n_splits <= 1) {
        const float inv = (gate ? __ldcg(gate + flat) : 1.0f) / l;
#pragma unroll
        for (int i = 0; i < LA_MAX_PAIRS; ++i) {
          const int col = (warp + LA_WARPS * i) * 16;
          if (col < dv) {
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2)
              *reinterpret_cast<__nv_bfloat162*>(out + flat * dv + col + h2 * 8 + qc) =
                  __floats2bfloat162_rn(o[mt][i][h2][half * 2] * inv, o[mt][i][h2][half * 2 + 1] * inv);
          }
        }
      } else {
        float* rec = scratch + (flat * n_splits + sp) * (dv + 2);
#pragma unroll
        for (int i = 0; i < LA_MAX_PAIRS; ++i) {
          const int col = (warp + LA_WARPS * i) * 16;
          if (col < dv) {
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2) {
              rec[col + h2 * 8 + qc] = o[mt][i][h2][half * 2];
              rec[col + h2 * 8 + qc + 1] = o[mt][i][h2][half * 2 + 1];
            }
          }
        }
        if (warp == 0 && (lane & 3) == 0) { rec[dv] = mx; rec[dv + 1] = l; }
      }
    }
  }
}

// out[row, :] from the per-chunk records of a row: with M the largest of the chunks' maxima and w_s = 2^(m_s - M),
// out = sum_s acc_s w_s / sum_s l_s w_s, both in chunk order.  A block that found no key for a row in its chunk
// (or that had no tile to work on) left nothing: such records are told by the chunk's first key lying beyond the row.
__global__ void latent_combine_kernel(const float* __restrict__ scratch, __nv_bfloat16* out, const int* __restrict__ row_start,
                                      const int* __restrict__ row_pos0, int H, int dv, int n_splits, int pages_per_chunk,
                                      const float* gate) {
  extern __shared__ float wsm[];                     // [n_splits] weights
  __shared__ float inv_l;
  pdl_wait();
  pdl_trigger();
  const int b = blockIdx.y;
  const int tok0 = __ldcg(row_start + b);
  const int F = (__ldcg(row_start + b + 1) - tok0) * H;
  const int f = blockIdx.x;
  if (f >= F) return;
  const int pos = __ldcg(row_pos0 + b) + f / H;
  const int used = min(n_splits, pos / (pages_per_chunk * LA_KEYS) + 1);   // chunks that hold a key this row sees
  const int64_t flat = (int64_t)tok0 * H + f;
  const int rec = dv + 2;
  const float* base = scratch + flat * n_splits * rec;
  for (int s = threadIdx.x; s < used; s += blockDim.x) wsm[s] = __ldcg(base + (int64_t)s * rec + dv);
  __syncthreads();
  float mx = -INFINITY;
  for (int s = 0; s < used; ++s) mx = fmaxf(mx, wsm[s]);
  __syncthreads();
  for (int s = threadIdx.x; s < used; s += blockDim.x) wsm[s] = la_exp2(wsm[s] - mx);
  __syncthreads();
  if (threadIdx.x == 0) {
    float ll = 0.0f;
    for (int s = 0; s < used; ++s) ll += __ldcg(base + (int64_t)s * rec + dv + 1) * wsm[s];
    inv_l = (gate ? __ldcg(gate + flat) : 1.0f) / ll;
  }
  __syncthreads();
  for (int d = threadIdx.x; d < dv; d += blockDim.x) {
    float aa = 0.0f;
#pragma unroll 4
    for (int s = 0; s < used; ++s) aa += __ldcg(base + (int64_t)s * rec + d) * wsm[s];
    out[flat * dv + d] = __float2bfloat16_rn(aa * inv_l);
  }
}

static size_t la_smem_bytes(int MT, int dk) {
  const size_t M = 16 * (size_t)MT;
  return ((M + 2 * LA_KEYS) * (dk + LA_PAD) + M * (LA_KEYS + LA_PAD)) * sizeof(__nv_bfloat16) +
         (2 * LA_WARPS * M + 3 * M) * sizeof(float);
}

template <int MT, bool PW>
static int la_launch(const void* q, void* out, const void* pool, const int* block_table, int bt_stride, const int* row_start,
                     const int* row_pos0, int B, int max_rows, int H, int dk, int dv, float scale, int pages_per_chunk,
                     int n_splits, float* scratch, const float* gate, cudaStream_t stream) {
  const size_t smem = la_smem_bytes(MT, dk);
  cudaError_t e = cudaFuncSetAttribute(attn_latent_kernel<MT, PW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("attn_latent: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    return (int)e;
  }
  dim3 grid(ceil_div(max_rows, 16 * MT), B, n_splits);
  launch_pdl(attn_latent_kernel<MT, PW>, grid, dim3(LA_THREADS + (PW ? 32 * LA_COPY_WARPS : 0)), smem, stream, static_cast<const __nv_bfloat16*>(q),
             static_cast<__nv_bfloat16*>(out), static_cast<const __nv_bfloat16*>(pool), block_table, bt_stride, row_start,
             row_pos0, H, dk, dv, scale * 1.4426950408889634f, pages_per_chunk, n_splits, scratch, gate);
  return launch_status("attn_latent");
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_attn_latent_row_tile(int dk, int max_rows) {
  // the largest tile of rows (in sixteens: 4, 3, 2 or 1) that a sequence's rows fill and whose shared memory fits; 0: none
  const size_t limit = 227 * 1024;
  static const int most = [] {                               // EXL3_LATENT_TILE=n: at most n sixteens (for measurements)
    const char* e = getenv("EXL3_LATENT_TILE");
    return e && e[0] >= '1' && e[0] <= '4' ? e[0] - '0' : 4;
  }();
  int mt = max_rows > 48 ? 4 : (max_rows > 32 ? 3 : (max_rows > 16 ? 2 : 1));
  if (mt > most) mt = most;
  while (mt >= 1 && la_smem_bytes(mt, dk) > limit) --mt;
  return mt;
}

extern "C" size_t exl3_attn_latent_scratch_bytes(int T, int H, int dv, int n_splits) {
  return n_splits <= 1 ? 0 : (size_t)T * H * n_splits * (dv + 2) * sizeof(float);
}

extern "C" int exl3_attn_latent(const void* q, void* out, const void* pool, const int* block_table, int bt_stride,
                                const int* row_start, const int* row_pos0, int B, int T, int max_new, int H, int dk, int dv,
                                int page, float scale, int pages_per_chunk, int n_splits, float* scratch,
                                size_t scratch_bytes, const float* gate, cudaStream_t stream) {
  if (B == 0 || T == 0) return 0;
  if (B < 0 || T < 0 || max_new < 1 || H < 1 || dk < 16 || dk % 16 != 0 || dv < 16 || dv % 16 != 0 || dv > dk ||
      dv > LA_WARPS * LA_MAX_PAIRS * 16 || page != LA_KEYS || n_splits < 1 || n_splits > 65535 ||
      (n_splits > 1 && pages_per_chunk < 1)) {
    set_error("attn_latent: bad sizes rows=%d tokens=%d heads=%d dk=%d dv=%d (multiples of 16, dv <= dk, dv <= %d) "
              "page=%d (must be %d) splits=%d", B, T, H, dk, dv, LA_WARPS * LA_MAX_PAIRS * 16, page, LA_KEYS, n_splits);
    return ERR_BAD_ARGUMENT;
  }
  if (!aligned16(q) || !aligned16(out) || !aligned16(pool)) {
    set_error("attn_latent: q, out and the pool must be 16-byte aligned");
    return ERR_ALIGNMENT;
  }
  if (exl3_attn_latent_scratch_bytes(T, H, dv, n_splits) > scratch_bytes) {
    set_error("attn_latent: scratch of %zu bytes is too small", scratch_bytes);
    return ERR_SCRATCH;
  }
  const int64_t max_rows64 = (int64_t)max_new * H;
  if (max_rows64 > 0x7fffffffLL || B > 65535) { set_error("attn_latent: grid too large"); return ERR_UNSUPPORTED; }
  const int max_rows = (int)max_rows64;
  const int mt = exl3_attn_latent_row_tile(dk, max_rows);
  int rc;
  if (mt == 3) rc = la_launch<3, false>(q, out, pool, block_table, bt_stride, row_start, row_pos0, B, max_rows, H, dk, dv, scale, pages_per_chunk, n_splits, scratch, gate, stream);
  else if (mt == 4) rc = la_launch<4, false>(q, out, pool, block_table, bt_stride, row_start, row_pos0, B, max_rows, H, dk, dv, scale, pages_per_chunk, n_splits, scratch, gate, stream);
  else if (mt == 2) rc = la_launch<2, true>(q, out, pool, block_table, bt_stride, row_start, row_pos0, B, max_rows, H, dk, dv, scale, pages_per_chunk, n_splits, scratch, gate, stream);
  else if (mt == 1) rc = la_launch<1, true>(q, out, pool, block_table, bt_stride, row_start, row_pos0, B, max_rows, H, dk, dv, scale, pages_per_chunk, n_splits, scratch, gate, stream);
  else { set_error("attn_latent: rows of %d features do not fit shared memory", dk); return ERR_UNSUPPORTED; }
  if (rc) return rc;
  if (n_splits > 1) {
    if (B > 65535) { set_error("attn_latent: too many sequences for the merge"); return ERR_UNSUPPORTED; }
    launch_pdl(latent_combine_kernel, dim3(max_rows, B), dim3(128), (size_t)n_splits * sizeof(float), stream,
               (const float*)scratch, static_cast<__nv_bfloat16*>(out), row_start, row_pos0, H, dv, n_splits,
               pages_per_chunk, gate);
    rc = launch_status("latent_combine");
  }
  return rc;
}
