// Token embedding plus a hashed second table.
//
//   h[t] = table[id_t] + extra[row_t]
//   row_t = (prev_t * mul_prev + id_t * mul_cur) mod buckets      for a token with a token before it
//         = buckets (the table's last row)                         for a sequence's first token
//
// The token before a row's first token of this step is part of the sequence's state: last_token[slot], which the
// block of that first token reads and then sets to the row's last token of the step (one thread does both, in that
// order, so a step of any length leaves the state right and no other block touches the entry).  The sum is float32.
#include "api.h"
#include "common.cuh"

namespace exl3 {

template <typename T>
__global__ void embed_hashed_kernel(const int* __restrict__ ids, const int* __restrict__ tok_pos,
                                    const int* __restrict__ tok_seq, const int* __restrict__ row_start,
                                    const int* __restrict__ slot_ids, const T* __restrict__ table,
                                    const T* __restrict__ extra, int buckets, long long mul_prev, long long mul_cur,
                                    int* last_token, float* __restrict__ h, int H, int V) {
  __shared__ int s_prev;
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int id = __ldcg(ids + t);
  const int pos = __ldcg(tok_pos + t);
  const int b = __ldcg(tok_seq + t);
  const int first = __ldcg(row_start + b), end = __ldcg(row_start + b + 1);
  if (threadIdx.x == 0) {
    int prev = -1;
    if (t == first) {
      int* st = last_token + __ldcg(slot_ids + b);
      prev = __ldcg(st);
      *st = __ldcg(ids + end - 1);
    } else {
      prev = __ldcg(ids + t - 1);
    }
    s_prev = prev;
  }
  __syncthreads();
  float* row = h + (int64_t)t * H;
  if (id < 0 || id >= V) {                       // refused on the host already; never read outside
    for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = 0.0f;
    return;
  }
  long long r = buckets;
  if (pos > 0) {
    r = ((long long)s_prev * mul_prev + (long long)id * mul_cur) % buckets;
    if (r < 0) r += buckets;
  }
  const T* a = table + (int64_t)id * H;
  const T* e = extra + (int64_t)r * H;
  for (int i = threadIdx.x; i < H; i += blockDim.x) row[i] = Elem<T>::load(a + i) + Elem<T>::load(e + i);
}

}  // namespace exl3

using namespace exl3;

extern "C" int exl3_embed_hashed(const int* ids, const int* tok_pos, const int* tok_seq, const int* row_start,
                                 const int* slot_ids, const void* table, const void* extra, int dtype, int buckets,
                                 long long mul_prev, long long mul_cur, int* last_token, float* h, int T, int H, int V,
                                 cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || H < 1 || V < 1 || buckets < 1 || last_token == nullptr) {
    set_error("embed_hashed: bad sizes T=%d H=%d V=%d buckets=%d", T, H, V, buckets);
    return ERR_BAD_ARGUMENT;
  }
  const int threads = H >= 1024 ? 256 : 128;
  if (dtype == DT_F32)
    launch_pdl(embed_hashed_kernel<float>, dim3(T), dim3(threads), 0, stream, ids, tok_pos, tok_seq, row_start, slot_ids,
               static_cast<const float*>(table), static_cast<const float*>(extra), buckets, mul_prev, mul_cur,
               last_token, h, H, V);
  else if (dtype == DT_BF16)
    launch_pdl(embed_hashed_kernel<__nv_bfloat16>, dim3(T), dim3(threads), 0, stream, ids, tok_pos, tok_seq, row_start,
               slot_ids, static_cast<const __nv_bfloat16*>(table), static_cast<const __nv_bfloat16*>(extra), buckets,
               mul_prev, mul_cur, last_token, h, H, V);
  else {
    set_error("embed_hashed: unsupported element type %d", dtype);
    return ERR_UNSUPPORTED;
  }
  return launch_status("embed_hashed");
}
