// Paged grouped-query attention, one warp per (query token, query head).
//
// The kernel of the true 32-bit path, and the fallback of the bfloat16 path for head
// sizes its tiled kernels do not take.  A query at position p of row r sees the keys of
// its request at positions lo..p (lo = max(0, p - window + 1) with a window, else 0), all
// read from the pages the row's block table names.  Keys are taken 32 at a time, chunks
// aligned to absolute positions (0-31, 32-63, ...), one key per lane; scores, the running
// maximum and sum, and the output accumulator are 32-bit.  The order of every sum depends
// only on the key's position, never on how the tokens were cut into steps or on what else
// is in the batch.
//
// The general entry takes queries of their own type (32-bit queries over a bfloat16 cache),
// keys and values of different head sizes, and a cap on the scores: s <- cap * tanh(s / cap)
// before the softmax.  A page holds its keys [nkv, page_size, hd] and then its values
// [nkv, page_size, vd]; with hd = vd that is the layout [2, nkv, page_size, hd] of the other
// attention kernels.  The output's rows may be wider than nh * vd (a slice of a joined buffer).
//
// Three further options.  `keep_first` > 0 beside a window: the first keep_first positions of a
// request stay visible to every later query (at their true positions); their chunks are walked
// first, in position order like the rest.  `values_are_keys`: a page holds keys only,
// [nkv, page_size, hd], and the values are those same vectors (vd = hd): attention over a cached
// latent.  `gate` (32-bit, [T, nh * vd] in rows of gate_stride): the output is multiplied element by
// element with sigmoid(gate).
//
// And three more.  `chunk` c > 0 (instead of a window): a query at position p sees the keys from p - p % c on, the
// run of c positions it lies in, runs counted from position 0.  `sinks` (32-bit, one number per query head): the
// softmax's denominator has one more term exp(sink) that has no key and no value and is not scaled or capped
// (a sink of 0 adds one).  `gate_group` g > 1: the gate holds one value per g output elements ([T, nh * vd / g];
// g = vd: one per head).
#include <math.h>
#include "common.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int MAX_HD = 512;

template <typename TQ, typename T>
__global__ void __launch_bounds__(WARPS * 32)
paged_attention_simple_kernel(const TQ* __restrict__ q, long long q_stride, const T* __restrict__ kv,
                              const int* __restrict__ block_tables, int bt_stride, const int* __restrict__ token_row,
                              const int* __restrict__ positions, T* __restrict__ out, long long out_stride, int n_tokens,
                              int nh, int nkv, int hd, int vd, int page_size, long long num_pages, float scale,
                              float softcap, int window, int R, int* status, int keep_first, int values_are_keys,
                              const float* gate, long long gate_stride, int chunk, const float* __restrict__ sinks,
                              int gate_group) {
  extern __shared__ float smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * WARPS + warp;
  if (w >= (long long)n_tokens * nh) return;
  const int t = (int)(w / nh), h = (int)(w - (long long)t * nh);
  const int g = h / (nh / nkv);
  float* qs = smem + warp * hd;
  const TQ* qp = q + (long long)t * q_stride + (long long)h * hd;
  for (int e = lane; e < hd; e += 32) qs[e] = to_f(qp[e]);
  __syncwarp();

  const int row = token_row[t];
  T* op = out + (long long)t * out_stride + (long long)h * vd;
  if (row < 0 || row >= R) {
    if (lane == 0) fmx_set_status(status, FMX_BAD_ROW, row, t);
    for (int e = lane; e < vd; e += 32) op[e] = from_f<T>(0.f);
    return;
  }
  const int pos = positions[t];
  const int* bt = block_tables + (long long)row * bt_stride;
  const int lo = window > 0 ? max(0, pos - window + 1) : (chunk > 0 && pos > 0 ? pos - pos % chunk : 0);
  const long long plane = values_are_keys ? 0 : (long long)nkv * page_size * hd;     // a page's keys, then its values
  const long long page_elems = (long long)nkv * page_size * (values_are_keys ? hd : hd + vd);
  // positions below `kept` are seen although the window has passed them
  const int kept = min(keep_first, lo);
  const int first_c = lo / 32, kept_c = kept > 0 ? (kept + 31) / 32 : 0;
  const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;

  float m = -INFINITY, l = 0.f;
  float acc[MAX_HD / 32];
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) acc[i] = 0.f;

  for (int c = kept_c > 0 ? 0 : first_c; c * 32 <= pos; ++c) {
    if (c >= kept_c && c < first_c) c = first_c;            // from the kept tokens straight to the window
    const int j = c * 32 + lane;
    bool valid = (j >= lo || j < kept) && j <= pos;
    float s = -INFINITY;
    long long vbase = 0;
    if (valid) {
      const int blk = j / page_size;
      const int page = blk < bt_stride ? bt[blk] : -1;
      if (page < 0 || page >= num_pages) {
        fmx_set_status(status, FMX_BAD_PAGE, page, t);
        valid = false;
      } else {
        const long long at = (long long)g * page_size + (j - blk * page_size);
        const long long kbase = (long long)page * page_elems + at * hd;
        vbase = (long long)page * page_elems + plane + at * vd;
        float dot = 0.f;
        for (int e = 0; e < hd; ++e) dot = fmaf(qs[e], to_f(kv[kbase + e]), dot);
        s = dot * scale;
        if (softcap > 0.f) s = softcap * tanhf(s * inv_cap);
      }
    }
    const float m_new = fmaxf(m, warp_max(s));
    if (m_new == -INFINITY) continue;
    const float p = valid ? expf(s - m_new) : 0.f;
    const float alpha = expf(m - m_new);
    l = l * alpha + warp_sum(p);
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; ++i) acc[i] *= alpha;
    for (int jj = 0; jj < 32; ++jj) {
      const float pj = __shfl_sync(0xffffffffu, p, jj);
      const long long vb = __shfl_sync(0xffffffffu, vbase, jj);
      if (pj == 0.f) continue;                // keys out of sight are never read
#pragma unroll
      for (int i = 0; i < MAX_HD / 32; ++i) {
        const int e = lane + 32 * i;
        if (e < vd) acc[i] = fmaf(pj, to_f(kv[vb + e]), acc[i]);
      }
    }
    m = m_new;
  }
  if (sinks != nullptr && m != -INFINITY) {      // the term without a value: the sums move to the larger maximum
    const float sk = sinks[h];
    const float m_new = fmaxf(m, sk);
    const float alpha = expf(m - m_new);
    l = l * alpha + expf(sk - m_new);
#pragma unroll
    for (int i = 0; i < MAX_HD / 32; ++i) acc[i] *= alpha;
  }
  const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
  for (int i = 0; i < MAX_HD / 32; ++i) {
    const int e = lane + 32 * i;
    if (e < vd) {
      float o = acc[i] * inv;
      if (gate != nullptr) o *= 1.0f / (1.0f + expf(-gate[(long long)t * gate_stride + ((long long)h * vd + e) / gate_group]));
      op[e] = from_f<T>(o);
    }
  }
}
}  // namespace

// q_dtype: the queries' type (FMX_F32 beside a bfloat16 cache, or the cache's own); dtype: the type of the
// cache and of the output; hd / vd: head sizes of keys and values; softcap <= 0: scores are not capped.
// keep_first, values_are_keys, gate, chunk, sinks, gate_group: see the head of the file (0, 0, null, 0, null, 1: none of them).
FMX_EXPORT int fmx_paged_attention_masked_ex(const void* q, long long q_stride, int q_dtype, const void* kv,
                                          const int* block_tables, int bt_stride, const int* token_row,
                                          const int* positions, void* out, long long out_stride, int n_tokens, int nh,
                                          int nkv, int hd, int vd, int page_size, long long num_pages, float scale,
                                          float softcap, int window, int R, int dtype, int* status, int keep_first,
                                          int values_are_keys, const float* gate, long long gate_stride, int chunk,
                                          const float* sinks, int gate_group, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  if (chunk < 0 || (chunk > 0 && window > 0) || gate_group < 1 || (gate != nullptr && (vd % gate_group) && gate_group != 1))
    return fmx_fail("fmx_paged_attention_general: bad chunk %d beside window %d, or gate group %d", chunk, window, gate_group);
  if (n_tokens < 0 || nh <= 0 || nkv <= 0 || nh % nkv || hd <= 0 || vd <= 0 || page_size <= 0)
    return fmx_fail("fmx_paged_attention_general: bad sizes T=%d nh=%d nkv=%d hd=%d vd=%d page=%d", n_tokens, nh, nkv, hd,
                    vd, page_size);
  if (hd > MAX_HD || vd > MAX_HD) return fmx_fail("fmx_paged_attention_general: head sizes %d / %d are above %d", hd, vd, MAX_HD);
  if (out_stride < (long long)nh * vd) return fmx_fail("fmx_paged_attention_general: output rows too narrow");
  const long long warps = (long long)n_tokens * nh;
  const long long grid = (warps + WARPS - 1) / WARPS;
  if (grid > 2147483647LL) return fmx_fail("fmx_paged_attention_general: batch too large");
  const size_t smem = (size_t)WARPS * hd * sizeof(float);
#define FMX_ATTN_SIMPLE(TQ, T)                                                                                        \
  paged_attention_simple_kernel<TQ, T><<<(unsigned)grid, WARPS * 32, smem, stream>>>(                                 \
      (const TQ*)q, q_stride, (const T*)kv, block_tables, bt_stride, token_row, positions, (T*)out, out_stride, n_tokens, \
      nh, nkv, hd, vd, page_size, num_pages, scale, softcap, window, R, status, keep_first, values_are_keys, gate,        \
      gate_stride, chunk, sinks, gate_group)
  if (values_are_keys && hd != vd) return fmx_fail("fmx_paged_attention_general: values that are the keys have the keys' width");
  if (keep_first < 0 || (gate != nullptr && gate_stride < (long long)nh * vd / gate_group))
    return fmx_fail("fmx_paged_attention_general: bad keep_first %d or gate rows too narrow", keep_first);
  if (dtype == FMX_F32 && q_dtype == FMX_F32)
    FMX_ATTN_SIMPLE(float, float);
  else if (dtype == FMX_BF16 && q_dtype == FMX_BF16)
    FMX_ATTN_SIMPLE(bf16, bf16);
  else if (dtype == FMX_BF16 && q_dtype == FMX_F32)
    FMX_ATTN_SIMPLE(float, bf16);
  else
    return fmx_fail("fmx_paged_attention_general: no kernel for queries of type %d over a cache of type %d", q_dtype, dtype);
#undef FMX_ATTN_SIMPLE
  FMX_LAUNCH_CHECK();
  return 0;
}

FMX_EXPORT int fmx_paged_attention_masked(const void* q, long long q_stride, int q_dtype, const void* kv,
                                          const int* block_tables, int bt_stride, const int* token_row,
                                          const int* positions, void* out, long long out_stride, int n_tokens, int nh,
                                          int nkv, int hd, int vd, int page_size, long long num_pages, float scale,
                                          float softcap, int window, int R, int dtype, int* status, int keep_first,
                                          int values_are_keys, const float* gate, long long gate_stride,
                                          cudaStream_t stream) {
  return fmx_paged_attention_masked_ex(q, q_stride, q_dtype, kv, block_tables, bt_stride, token_row, positions, out, out_stride,
                                       n_tokens, nh, nkv, hd, vd, page_size, num_pages, scale, softcap, window, R, dtype, status,
                                       keep_first, values_are_keys, gate, gate_stride, 0, nullptr, 1, stream);
}

FMX_EXPORT int fmx_paged_attention_general(const void* q, long long q_stride, int q_dtype, const void* kv,
                                           const int* block_tables, int bt_stride, const int* token_row,
                                           const int* positions, void* out, long long out_stride, int n_tokens, int nh,
                                           int nkv, int hd, int vd, int page_size, long long num_pages, float scale,
                                           float softcap, int window, int R, int dtype, int* status,
                                           cudaStream_t stream) {
  return fmx_paged_attention_masked(q, q_stride, q_dtype, kv, block_tables, bt_stride, token_row, positions, out, out_stride,
                                    n_tokens, nh, nkv, hd, vd, page_size, num_pages, scale, softcap, window, R, dtype, status,
                                    0, 0, nullptr, 0, stream);
}

FMX_EXPORT int fmx_paged_attention_simple(const void* q, long long q_stride, const void* kv, const int* block_tables,
                                          int bt_stride, const int* token_row, const int* positions, void* out,
                                          int n_tokens, int nh, int nkv, int hd, int page_size, long long num_pages,
                                          float scale, int window, int R, int dtype, int* status,
                                          cudaStream_t stream) {
  return fmx_paged_attention_general(q, q_stride, dtype, kv, block_tables, bt_stride, token_row, positions, out,
                                     (long long)nh * hd, n_tokens, nh, nkv, hd, hd, page_size, num_pages, scale, 0.f,
                                     window, R, dtype, status, stream);
}
