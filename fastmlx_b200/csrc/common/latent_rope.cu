// Latent attention with a rotated key part beside the latent: what a token leaves in the cache, and the rotated
// parts of its queries.
//
// A token's down-projection d [r + R] (32-bit) becomes its cache row [c | k_rot]: c = d[:r] divided by its root mean
// square (eps inside the root) times a weight; k_rot = d[r:] rotated by the token's position, pairs (i, i + R/2),
// angle position * inv_freq[i].  A query head is [D unrotated | R rotated] values: the rotated part, turned the same
// way, goes to q_lat[t, h, r : r + R] in 32-bit, behind the place where the head's unrotated part is carried into
// the latent's space by another kernel.  Angles, sines, cosines, the sum of squares and the division are 32-bit.
// One block per token.  R = 0: only the latent's norm and store.
#include "common.cuh"

namespace {
constexpr int LRP_THREADS = 128;

template <typename TQ, typename T>
__global__ void __launch_bounds__(LRP_THREADS)
latent_rope_prepare_kernel(const TQ* q, long long q_stride, const float* dkv, long long dkv_stride, const int* positions,
                           const float* __restrict__ inv_freq, const float* __restrict__ norm_w, float eps,
                           const long long* slot_mapping, T* kv, long long max_rows, float* q_lat, int H, int D, int R,
                           int r, int q_off, int* status) {
  extern __shared__ float sc[];                  // [R/2] sines, [R/2] cosines
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int half = R / 2, row = r + R;
  float* sn = sc;
  float* cs = sc + half;
  const float pos = (float)positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &sn[j], &cs[j]);
  float ss = 0.f;
  const float* dp = dkv != nullptr ? dkv + (long long)t * dkv_stride : nullptr;
  long long slot = (kv != nullptr && slot_mapping != nullptr && dp != nullptr) ? slot_mapping[t] : -1;
  if (slot >= max_rows) {
    if (threadIdx.x == 0) fmx_set_status(status, FMX_BAD_SLOT, slot, t);
    slot = -1;
  }
  if (slot >= 0)
    for (int e = threadIdx.x; e < r; e += blockDim.x) ss = fmaf(dp[e], dp[e], ss);
  ss = block_sum<LRP_THREADS>(ss);               // (its barriers also publish the sines and cosines)
  if (q_lat != nullptr) {
    const TQ* qp = q + (long long)t * q_stride;
    const int q_row = q_off + R;                 // a head of q_lat: q_off values that are not written here, then the rotated part
    float* out = q_lat + (long long)t * H * q_row;
    for (int i = threadIdx.x; i < H * half; i += blockDim.x) {
      const int h = i / half, j = i - h * half;
      const TQ* src = qp + (long long)h * (D + R) + D;
      float x, y;
      rope_pair(to_f(src[j]), to_f(src[j + half]), sn[j], cs[j], x, y);
      out[(long long)h * q_row + q_off + j] = x;
      out[(long long)h * q_row + q_off + half + j] = y;
    }
  }
  if (slot < 0) return;
  T* dst = kv + slot * row;
  const float rstd = 1.0f / sqrtf(ss / (float)r + eps);
  for (int e = threadIdx.x; e < r; e += blockDim.x) dst[e] = from_f<T>(dp[e] * rstd * norm_w[e]);
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float x, y;
    rope_pair(dp[r + j], dp[r + half + j], sn[j], cs[j], x, y);
    dst[r + j] = from_f<T>(x);
    dst[r + half + j] = from_f<T>(y);
  }
}
}  // namespace

// q [T, >= H*(D+R)] of q_dtype (null with q_lat null: nothing of the queries is done); dkv [T, >= r+R] 32-bit and kv
// (rows of r + R values of `dtype`, max_rows of them) may be null: a layer that reads another layer's cache.  q_lat
// [T, H, q_off + R] takes the rotated query parts behind the first q_off values of a head (q_off < 0: r).
FMX_EXPORT int fmx_latent_rope_prepare(const void* q, long long q_stride, int q_dtype, const float* dkv, long long dkv_stride,
                                       const int* positions, const float* inv_freq, const float* norm_w, float eps,
                                       const long long* slot_mapping, void* kv, long long max_rows, int dtype, float* q_lat,
                                       int T, int H, int D, int R, int r, int q_off, int* status, cudaStream_t stream) {
  if (T == 0) return 0;
  if (q_off < 0) q_off = r;
  if (T < 0 || H <= 0 || D <= 0 || R < 0 || (R & 1) || r <= 0)
    return fmx_fail("fmx_latent_rope_prepare: bad sizes T=%d H=%d D=%d R=%d r=%d", T, H, D, R, r);
  if (R > 0 && inv_freq == nullptr) return fmx_fail("fmx_latent_rope_prepare: R=%d needs a frequency table", R);
  if (kv != nullptr && (dkv == nullptr || norm_w == nullptr || slot_mapping == nullptr || dkv_stride < r + R))
    return fmx_fail("fmx_latent_rope_prepare: a cache needs the down-projection, its norm's weight and the slots");
  if (q_lat != nullptr && (q == nullptr || q_stride < (long long)H * (D + R)))
    return fmx_fail("fmx_latent_rope_prepare: query rows too narrow");
  const size_t smem = (size_t)(R > 0 ? R : 1) * sizeof(float);
#define FMX_LRP(TQ, TKV)                                                                                               \
  fmx_launch(latent_rope_prepare_kernel<TQ, TKV>, dim3(T), dim3(LRP_THREADS), smem, stream, (const TQ*)q, q_stride, dkv, \
             dkv_stride, positions, inv_freq, norm_w, eps, slot_mapping, (TKV*)kv, max_rows, R > 0 ? q_lat : (float*)nullptr, \
             H, D, R, r, q_off, status)
  if (q_dtype == FMX_F32 && dtype == FMX_F32)
    FMX_LRP(float, float);
  else if (q_dtype == FMX_BF16 && dtype == FMX_BF16)
    FMX_LRP(bf16, bf16);
  else if (q_dtype == FMX_F32 && dtype == FMX_BF16)
    FMX_LRP(float, bf16);
  else
    return fmx_fail("fmx_latent_rope_prepare: no kernel for queries of type %d and a cache of type %d", q_dtype, dtype);
#undef FMX_LRP
  FMX_LAUNCH_CHECK();
  return 0;
}
