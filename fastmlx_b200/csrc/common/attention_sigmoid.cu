// Paged attention without a softmax, whose heads' weights are mixed before they meet the values.
//
// A query at position p of head g gives a visible key j (j <= p, and j > p - window with a window) the weight
//     w_g(p, j) = sigmoid(cap(scale * q_g . k_kv(g)(j)) + b_g),      cap(s) = c tanh(s / c) where c > 0,
// with one number b_g per head; weights are not normalised over the keys.  The heads' weights are then mixed by
// a square matrix M, w'_h = sum_g M[h, g] w_g, and head h applies w'_h to the values of its own key/value head.
// Since nothing is normalised the mix commutes with the sum over keys:
//     o_h(p) = sum_g M[h, g] A[g, kv(h)](p),     A[g, c](p) = sum_j w_g(p, j) v_c(j),
// so the work is done in two kernels.
//
//   sigmoid_attention   one warp per (token, query head g, value head c): A[g, c] in 32-bit.  Keys are taken 32 at a
//                       time, chunks aligned to absolute positions, one key per lane; the 32 weights then meet the
//                       values key by key.  The order of every sum depends on the key's position alone, never on how
//                       the tokens were cut into steps or on what else is in the batch.
//   head_mix            one block per token: o_h = sum_g M[h, g] A[g, kv(h)], g in order, out in the run's type.
//
// Pages hold their keys [nkv, page_size, hd] and then their values [nkv, page_size, vd], as for the other kernels.
#include <math.h>
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_HD = 512;

template <typename TQ, typename T>
__global__ void __launch_bounds__(WARPS * 32)
sigmoid_attention_kernel(const TQ* q, long long q_stride, const T* kv, const int* block_tables, int bt_stride,
                         const int* token_row, const int* positions, float* part, int n_tokens, int nh, int nkv, int hd,
                         int vd, int page_size, long long num_pages, float scale, float softcap, int window, int R,
                         const float* __restrict__ head_bias, int* status) {
  extern __shared__ float smem[];
  pdl_wait();
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * WARPS + warp;
  if (w >= (long long)n_tokens * nh * nkv) return;
  const int t = (int)(w / ((long long)nh * nkv));
  const int rem = (int)(w - (long long)t * nh * nkv);
  const int h = rem / nkv, c = rem - h * nkv;    // query head, value head
  const int g = h / (nh / nkv);                  // the query head's key head
  float* qs = smem + warp * hd;
  const TQ* qp = q + (long long)t * q_stride + (long long)h * hd;
  for (int e = lane; e < hd; e += 32) qs[e] = to_f(qp[e]);
  __syncwarp();

  float* op = part + (((long long)t * nh + h) * nkv + c) * vd;
  const int row = token_row[t];
  if (row < 0 || row >= R) {
    if (lane == 0) fmx_set_status(status, FMX_BAD_ROW, row, t);
    for (int e = lane; e < vd; e += 32) op[e] = 0.f;
    return;
  }
  const int pos = positions[t];
  const int* bt = block_tables + (long long)row * bt_stride;
  const int lo = window > 0 ? max(0, pos - window + 1) : 0;
  const long long plane = (long long)nkv * page_size * hd;
  const long long page_elems = (long long)nkv * page_size * (hd + vd);
  const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;
  const float hb = head_bias != nullptr ? head_bias[h] : 0.f;

  float acc[MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) acc[i] = 0.f;

  for (int ch = lo / 32; ch * 32 <= pos; ++ch) {
    const int j = ch * 32 + lane;
    const bool valid = j >= lo && j <= pos;
    float p = 0.f;
    long long vbase = 0;
    if (valid) {
      const int blk = j / page_size;
      const int page = blk < bt_stride ? bt[blk] : -1;
      if (page < 0 || page >= num_pages) {
        fmx_set_status(status, FMX_BAD_PAGE, page, t);
      } else {
        const int at = j - blk * page_size;
        const long long kbase = (long long)page * page_elems + ((long long)g * page_size + at) * hd;
        vbase = (long long)page * page_elems + plane + ((long long)c * page_size + at) * vd;
        float dot = 0.f;
        for (int e = 0; e < hd; ++e) dot = fmaf(qs[e], to_f(kv[kbase + e]), dot);
        float s = dot * scale;
        if (softcap > 0.f) s = softcap * tanhf(s * inv_cap);
        p = 1.0f / (1.0f + expf(-(s + hb)));
      }
    }
    for (int jj = 0; jj < 32; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long vb = __shfl_sync(0xffffffffu, vbase, jj);
      if (pj == 0.f) continue;                   // keys out of sight are never read
#pragma unroll
      for (int i = 0; i < MAX_HD / 32; ++i) {
        const int e = lane + 32 * i;
        if (e < vd) acc[i] = fmaf(pj, to_f(kv[vb + e]), acc[i]);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) {
    const int e = lane + 32 * i;
    if (e < vd) op[e] = acc[i];
  }
}

// part [T, nh, nkv, vd] 32-bit; mix [nh, nh] (row: the head that receives); out rows of out_stride elements.
template <typename T>
__global__ void __launch_bounds__(128)
head_mix_kernel(const float* part, const float* __restrict__ mix, T* out, long long out_stride, int nh, int nkv, int vd) {
  pdl_wait();
  pdl_trigger();
  const long long t = blockIdx.x;
  const float* pt = part + t * nh * nkv * vd;
  const int per = nh / nkv;
  for (int it = threadIdx.x; it < nh * vd; it += blockDim.x) {
    const int h = it / vd, e = it - h * vd;
    const int c = h / per;
    float o = 0.f;
    for (int g = 0; g < nh; ++g) o = fmaf(mix[h * nh + g], pt[((long long)g * nkv + c) * vd + e], o);
    out[t * out_stride + it] = from_f<T>(o);
  }
}
}  // namespace

// q_dtype: the queries' type (FMX_F32 beside a bfloat16 cache, or the cache's own); dtype: the cache's type.
// part: [T, nh, nkv, vd] floats, A[g, c] of every token.  softcap <= 0: scores are not capped; window 0: every earlier
// key is seen; head_bias null: no number is added to the scores.
FMX_EXPORT int fmx_sigmoid_attention(const void* q, long long q_stride, int q_dtype, const void* kv, const int* block_tables,
                                     int bt_stride, const int* token_row, const int* positions, float* part, int n_tokens,
                                     int nh, int nkv, int hd, int vd, int page_size, long long num_pages, float scale,
                                     float softcap, int window, int R, int dtype, const float* head_bias, int* status,
                                     cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  if (n_tokens < 0 || nh <= 0 || nkv <= 0 || nh % nkv || hd <= 0 || vd <= 0 || page_size <= 0 || window < 0)
    return fmx_fail("fmx_sigmoid_attention: bad sizes T=%d nh=%d nkv=%d hd=%d vd=%d page=%d", n_tokens, nh, nkv, hd, vd, page_size);
  if (hd > MAX_HD || vd > MAX_HD) return fmx_fail("fmx_sigmoid_attention: head sizes %d / %d are above %d", hd, vd, MAX_HD);
  const long long warps = (long long)n_tokens * nh * nkv;
  const long long grid = (warps + WARPS - 1) / WARPS;
  if (grid > 2147483647LL) return fmx_fail("fmx_sigmoid_attention: batch too large");
  const size_t smem = (size_t)WARPS * hd * sizeof(float);
#define FMX_SIGA(TQ, T)                                                                                                  \
  fmx_launch(sigmoid_attention_kernel<TQ, T>, dim3((unsigned)grid), dim3(WARPS * 32), smem, stream, (const TQ*)q, q_stride, \
             (const T*)kv, block_tables, bt_stride, token_row, positions, part, n_tokens, nh, nkv, hd, vd, page_size,     \
             num_pages, scale, softcap, window, R, head_bias, status)
  if (dtype == FMX_F32 && q_dtype == FMX_F32) FMX_SIGA(float, float);
  else if (dtype == FMX_BF16 && q_dtype == FMX_BF16) FMX_SIGA(bf16, bf16);
  else if (dtype == FMX_BF16 && q_dtype == FMX_F32) FMX_SIGA(float, bf16);
  else return fmx_fail("fmx_sigmoid_attention: no kernel for queries of type %d over a cache of type %d", q_dtype, dtype);
#undef FMX_SIGA
  FMX_LAUNCH_CHECK();
  return 0;
}

FMX_EXPORT int fmx_head_mix(const float* part, const float* mix, void* out, long long out_stride, int dtype, int n_tokens,
                            int nh, int nkv, int vd, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  if (n_tokens < 0 || nh <= 0 || nkv <= 0 || nh % nkv || vd <= 0 || out_stride < (long long)nh * vd)
    return fmx_fail("fmx_head_mix: bad sizes T=%d nh=%d nkv=%d vd=%d", n_tokens, nh, nkv, vd);
  if (dtype == FMX_F32)
    fmx_launch(head_mix_kernel<float>, dim3(n_tokens), dim3(128), 0, stream, part, mix, (float*)out, out_stride, nh, nkv, vd);
  else if (dtype == FMX_BF16)
    fmx_launch(head_mix_kernel<bf16>, dim3(n_tokens), dim3(128), 0, stream, part, mix, (bf16*)out, out_stride, nh, nkv, vd);
  else
    return fmx_fail("fmx_head_mix: unknown dtype %d", dtype);
  FMX_LAUNCH_CHECK();
  return 0;
}
