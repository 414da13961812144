// Attention over latent rows on the tensor cores (bfloat16): every head of a token reads the same cached row
// [ c (values, dv features) | rotated key part | padding ] of dk features, so the query rows of one sequence,
// flattened over (token, head), are ONE matrix Q [rows, dk] against ONE key matrix K [keys, dk] whose leading dv
// columns are also the values:
//
//   S = Q K^T * scale,  row f = (token f / H, head f % H) sees keys j <= pos0 + f / H,  O = softmax(S) K[:, :dv]
//
// One kernel serves prompts, portions of prompts and single tokens.  A block of eight warps takes a tile of
// 16 * MT consecutive rows of one sequence and walks the sequence's pages (64 keys, one page a step, the next page
// on its way while this one is worked on).  All warps share all rows: for the scores a warp owns 8 of
// the page's 64 keys (its B fragments serve every row tile), for the output it owns every eighth 16-column slice
// of the values (its B fragments, read transposed out of the very tile the keys came from, again serve every row
// tile).  Row maxima and sums meet in shared memory; the running maximum, the running sum and the output
// accumulators are float32, the probabilities are rounded to bfloat16 for the second product.  With n_splits > 1 a
// block takes only the pages of one chunk (chunks are aligned to absolute positions) and leaves a record
// [dv sums, maximum, sum] per row and chunk, which latent_combine_kernel merges in chunk order.
//
// A page of keys comes as TMA tile copies (boxes of 64 keys x 64 features, 128-byte swizzle, which ldmatrix then
// follows) that one thread asks for a page ahead; they report to an mbarrier per buffer, and every wait on one is
// bounded (a block that gives up sets a flag for the host, exl3_attn_latent_status, and leaves).
//
// Exponentials are base 2: scores carry scale * log2(e), maxima are in those units everywhere.
#include "api.h"
#include "common.cuh"

#include <cuda.h>
#include <math.h>
#include <stdlib.h>

namespace exl3 {

constexpr int LA_WARPS = 8;
constexpr int LA_THREADS = LA_WARPS * 32;
constexpr int LA_KEYS = 64;                // keys per step: one page
constexpr int LA_PAD = 8;                  // elements added to a shared-memory row: 16-byte pieces of consecutive rows fall into different banks
constexpr int LA_MAX_PAIRS = 4;            // 16-column slices of the values per warp: dv <= 8 * 4 * 16 = 512

__device__ inline void la_ldmatrix_x4(uint32_t (&r)[4], const void* p) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ inline void la_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ inline float la_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Bounded wait for a page's copies (false when they did not land within the limit; the host reads the flag).
constexpr uint32_t LA_WAIT_LIMIT = 1u << 24;
static __device__ int g_la_error = 0;
__device__ inline uint32_t la_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ inline bool la_mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < LA_WAIT_LIMIT; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
// Address of the 16-byte piece that holds (key row, feature col) of a key tile as the copies lay it out: boxes of 64
// features, 8 KB each, a row of a box 128 bytes, its 16-byte pieces swizzled by the row (128-byte swizzle).
__device__ inline uint32_t la_key_addr(uint32_t tile, int row, int col) {
  return tile + (uint32_t)(col >> 6) * 8192u + (uint32_t)row * 128u + (uint32_t)((((col >> 3) & 7) ^ (row & 7)) << 4);
}
__device__ inline void la_ldsm_x2(uint32_t (&r)[2], uint32_t a) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ inline void la_ldsm_x4_trans(uint32_t (&r)[4], uint32_t a) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}

template <int MT>
__global__ void __launch_bounds__(LA_THREADS, 1)
attn_latent_kernel(const __grid_constant__ CUtensorMap map_k, const __nv_bfloat16* q, __nv_bfloat16* out,
                   const int* __restrict__ block_table, int bt_stride, const int* __restrict__ row_start,
                   const int* __restrict__ row_pos0, int H, int dk, int dv, float scale_log2, int pages_per_chunk,
                   int n_splits, float* scratch, const float* gate) {
  constexpr int M = 16 * MT;
  extern __shared__ unsigned char la_smem_raw[];
  const int ldk = dk + LA_PAD;                      // elements per shared-memory row of Q
  constexpr int ldp = LA_KEYS + LA_PAD;
  const int boxes = (dk + 63) >> 6;                 // copies per page: 64 keys x 64 features each
  const uint32_t tile_bytes = (uint32_t)boxes * 8192u;
  // two key tiles first, on a 1 KB boundary (the swizzle's unit); then Q, P, the statistics, two mbarriers
  unsigned char* base = la_smem_raw + ((1024u - (la_u32(la_smem_raw) & 1023u)) & 1023u);
  const uint32_t Ks = la_u32(base);
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(base + 2 * (size_t)tile_bytes);
  __nv_bfloat16* Ps = Qs + (size_t)M * ldk;
  float* red_max = reinterpret_cast<float*>(Ps + (size_t)M * ldp);   // [LA_WARPS][M]
  float* red_sum = red_max + LA_WARPS * M;          // [LA_WARPS][M]
  float* m_run = red_sum + LA_WARPS * M;            // [M]
  float* l_run = m_run + M;                         // [M]
  float* corr = l_run + M;                          // [M]
  uint64_t* bars = reinterpret_cast<uint64_t*>(corr + M + (M & 1));  // [2], 8-byte aligned

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

  // One thread asks for a page: `boxes` tile copies that report their bytes to the buffer's mbarrier.  A page that
  // is not there (never the case for a key that a row sees) reads page 0; features beyond dk come as zeros.
  auto ask = [&](int pg, int buf) {
    const uint32_t bar = la_u32(bars + buf);
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(tile_bytes) : "memory");
    const int row0 = (pg < 0 ? 0 : pg) * LA_KEYS;
    for (int j = 0; j < boxes; ++j)
      asm volatile(
          "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
          ::"r"(Ks + (uint32_t)buf * tile_bytes + (uint32_t)j * 8192u), "l"(&map_k), "r"(bar), "r"(j * 64), "r"(row0)
          : "memory");
  };
  if (tid == 0) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(la_u32(bars)));
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(la_u32(bars + 1)));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    if (page_lo <= page_hi) ask(__ldcg(bt + page_lo), 0);
  }
  // page numbers are fetched one step before the copies that need them
  int pg_next = (tid == 0 && page_lo + 1 <= page_hi) ? __ldcg(bt + page_lo + 1) : -1;
  // the queries of the tile; rows beyond the sequence's are zero
  for (int i = tid; i < M * vecs; i += LA_THREADS) {
    const int r = i / vecs, c = (i - r * vecs) * 8;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < rows) v = __ldcg(reinterpret_cast<const uint4*>(q + ((int64_t)tok0 * H + f0 + r) * dk + c));
    *reinterpret_cast<uint4*>(Qs + (size_t)r * ldk + c) = v;
  }
  if (tid < M) { m_run[tid] = -INFINITY; l_run[tid] = 0.0f; }
  __syncthreads();                                           // Q, the statistics and the mbarriers are set up

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
  bool fine = true;

  for (int pi = page_lo; pi <= page_hi; ++pi) {
    const int buf = (pi - page_lo) & 1;
    // this page's keys have landed (every thread looks for itself; the block then agrees on what it saw)
    const bool landed = la_mbar_wait(la_u32(bars + buf), ((pi - page_lo) >> 1) & 1);
    if (!__syncthreads_and(landed)) { fine = false; break; }
    if (tid == 0 && pi + 1 <= page_hi) {
      ask(pg_next, buf ^ 1);                                 // that buffer's last readers passed the page's last barrier
      pg_next = pi + 2 <= page_hi ? __ldcg(bt + pi + 2) : -1;
    }
    const uint32_t Kt = Ks + (uint32_t)buf * tile_bytes;

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
          la_ldsm_x2(bfr[which][u], la_key_addr(Kt, bk_row, kk + bk_col));
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
    __syncthreads();
    if (tid < M) {
      float mx = red_max[tid];
#pragma unroll
      for (int w = 1; w < LA_WARPS; ++w) mx = fmaxf(mx, red_max[w * M + tid]);
      const float mo = m_run[tid], mn = fmaxf(mo, mx);
      corr[tid] = mn == -INFINITY ? 1.0f : la_exp2(mo - mn);      // exp2(-inf) = 0 the first time
      m_run[tid] = mn;
    }
    __syncthreads();
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
    __syncthreads();
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
        if (col < dv) la_ldsm_x4_trans(vf[i], la_key_addr(Kt, kk + bv_row, col + bv_col));
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
    __syncthreads();                                         // P, the statistics and this key tile are free again
  }
  if (!fine) {
    if (tid == 0) atomicExch(&g_la_error, 1);                // the host reads this; the rows get what was summed so far
  }
  __syncthreads();                                           // the statistics, also when the chunk held no page

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
  const size_t tile = (size_t)((dk + 63) / 64) * 8192;       // a page of keys: boxes of 64 x 64
  return 1024 + 2 * tile + (M * (dk + LA_PAD) + M * (LA_KEYS + LA_PAD)) * sizeof(__nv_bfloat16) +
         (2 * LA_WARPS * M + 3 * M + 2) * sizeof(float) + 2 * sizeof(uint64_t);
}

typedef CUresult (*LaEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static LaEncodeFn la_encode_fn() {
  static LaEncodeFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    return reinterpret_cast<LaEncodeFn>(p);
  }();
  return fn;
}
// The pool as [pages * 64 rows, dk features] bfloat16; boxes of 64 features x 64 rows, 128-byte swizzle, zeros beyond dk.
static int la_make_map(CUtensorMap* map, const void* pool, int64_t rows, int dk) {
  LaEncodeFn fn = la_encode_fn();
  if (!fn) { set_error("attn_latent: the driver has no cuTensorMapEncodeTiled"); return ERR_UNSUPPORTED; }
  const cuuint64_t dims[2] = {(cuuint64_t)dk, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)dk * 2};
  const cuuint32_t box[2] = {64, (cuuint32_t)LA_KEYS};
  const cuuint32_t elem[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(pool), dims, strides, box, elem,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("attn_latent: cuTensorMapEncodeTiled failed with %d", (int)r); return ERR_BAD_ARGUMENT; }
  return 0;
}

template <int MT>
static int la_launch(const CUtensorMap& map, const void* q, void* out, const int* block_table, int bt_stride,
                     const int* row_start, const int* row_pos0, int B, int max_rows, int H, int dk, int dv, float scale,
                     int pages_per_chunk, int n_splits, float* scratch, const float* gate, cudaStream_t stream) {
  const size_t smem = la_smem_bytes(MT, dk);
  cudaError_t e = cudaFuncSetAttribute(attn_latent_kernel<MT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_error("attn_latent: %zu bytes of shared memory refused: %s", smem, cudaGetErrorString(e));
    return (int)e;
  }
  dim3 grid(ceil_div(max_rows, 16 * MT), B, n_splits);
  launch_pdl(attn_latent_kernel<MT>, grid, dim3(LA_THREADS), smem, stream, map, static_cast<const __nv_bfloat16*>(q),
             static_cast<__nv_bfloat16*>(out), block_table, bt_stride, row_start, row_pos0, H, dk, dv,
             scale * 1.4426950408889634f, pages_per_chunk, n_splits, scratch, gate);
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

// 1 when a block gave up waiting for a page's copies since the last call (its rows are then not to be trusted); clears it.
extern "C" int exl3_attn_latent_status() {
  int v = 0;
  cudaMemcpyFromSymbol(&v, g_la_error, sizeof(int));
  if (v) { int z = 0; cudaMemcpyToSymbol(g_la_error, &z, sizeof(int)); }
  return v;
}

extern "C" int exl3_attn_latent(const void* q, void* out, const void* pool, int64_t pool_pages, const int* block_table, int bt_stride,
                                const int* row_start, const int* row_pos0, int B, int T, int max_new, int H, int dk, int dv,
                                int page, float scale, int pages_per_chunk, int n_splits, float* scratch,
                                size_t scratch_bytes, const float* gate, cudaStream_t stream) {
  if (B == 0 || T == 0) return 0;
  if (B < 0 || T < 0 || max_new < 1 || H < 1 || dk < 16 || dk % 16 != 0 || dv < 16 || dv % 16 != 0 || dv > dk ||
      dv > LA_WARPS * LA_MAX_PAIRS * 16 || page != LA_KEYS || n_splits < 1 || n_splits > 65535 || pool_pages < 1 ||
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
  CUtensorMap map;
  int rc = la_make_map(&map, pool, pool_pages * LA_KEYS, dk);
  if (rc) return rc;
#define EXL3_LA(MT) la_launch<MT>(map, q, out, block_table, bt_stride, row_start, row_pos0, B, max_rows, H, dk, dv, scale, \
                                  pages_per_chunk, n_splits, scratch, gate, stream)
  if (mt == 4) rc = EXL3_LA(4);
  else if (mt == 3) rc = EXL3_LA(3);
  else if (mt == 2) rc = EXL3_LA(2);
  else if (mt == 1) rc = EXL3_LA(1);
  else { set_error("attn_latent: rows of %d features do not fit shared memory", dk); return ERR_UNSUPPORTED; }
#undef EXL3_LA
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
