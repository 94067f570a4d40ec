// Retention: linear attention with one fixed decay per head and no softmax or denominator.
//
// Per head h, with q, k (size D) and v (size P), a token does
//     S <- decay_h S + k v^T;   o = S^T q,
// S [D, P] in 32-bit in a state slot of the request, carried from step to step.  That is the state-space
// recurrence of ssm.cu with a step size of 1, a decay that no token changes, as many groups as heads and no skip
// term, so the recurrence itself runs on ssm_scan; the two kernels here stand in front of it and behind it.
//
//   retention_prepare    per token: q and k of every head rotated over their first `rot` dimensions (dimension i
//                        paired with i + rot/2; angle, sine and cosine in 32-bit), k multiplied by `k_scale` after
//                        the rotation; out [T, C] in 32-bit, C = H*P + 2*H*D, laid out as the scan takes its
//                        operands: v | k | q; and per head a step size of 1 and the head's decay, [T, 2H].
//   retention_gate_norm  one warp per (token, head): o divided by its root mean square over the head (no weight),
//                        times silu(gate), out in the run's type.
//
// Everything is 32-bit but the projection that comes in and the activations that go out.
#include <math.h>
#include "common.cuh"

namespace {
// proj [T, stride]: q (H*D) | k (H*D) | v (H*P)
template <typename T>
__global__ void __launch_bounds__(128)
retention_prepare_kernel(const T* proj, long long stride, const int* positions, const float* __restrict__ inv_freq,
                         const float* __restrict__ decay, float* out_xbc, float* out_dd, int H, int D, int P, int rot,
                         float k_scale) {
  extern __shared__ float smem[];               // [rot/2] sines, [rot/2] cosines
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int half = rot / 2;
  float* sn = smem;
  float* cs = smem + half;
  const float pos = (float)positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &sn[j], &cs[j]);
  __syncthreads();
  const T* row = proj + (long long)t * stride;
  const int inner = H * P, HD = H * D, C = inner + 2 * HD;
  float* ox = out_xbc + (long long)t * C;
  for (int e = threadIdx.x; e < inner; e += blockDim.x) ox[e] = to_f(row[2 * HD + e]);
  // one thread per (q or k, head, pair or unrotated dimension)
  const int per_head = D - half;                 // `half` pairs and D - rot dimensions that pass
  for (int it = threadIdx.x; it < 2 * H * per_head; it += blockDim.x) {
    const int which = it / (H * per_head);       // 0: q, 1: k
    const int rem = it - which * H * per_head;
    const int h = rem / per_head, j = rem - h * per_head;
    const T* src = row + (long long)which * HD + (long long)h * D;
    float* dst = ox + inner + (long long)(which == 0 ? HD : 0) + (long long)h * D;      // k first, then q
    const float mul = which == 0 ? 1.0f : k_scale;
    if (j < half) {
      float x, y;
      rope_pair(to_f(src[j]), to_f(src[j + half]), sn[j], cs[j], x, y);
      dst[j] = x * mul;
      dst[j + half] = y * mul;
    } else {
      const int e = j + half;
      dst[e] = to_f(src[e]) * mul;
    }
  }
  float* od = out_dd + (long long)t * 2 * H;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    od[h] = 1.0f;
    od[H + h] = decay[h];
  }
}

template <typename TG, typename T>
__global__ void __launch_bounds__(128)
retention_gate_norm_kernel(const float* o, const TG* gate, long long g_stride, T* out, long long out_stride, long long n_heads,
                           int H, int P, float eps) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const long long w = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (w >= n_heads) return;
  const long long t = w / H;
  const int h = (int)(w - t * H);
  const float* op = o + w * P;
  float ss = 0.f;
  for (int e = lane; e < P; e += 32) ss = fmaf(op[e], op[e], ss);
  const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)P + eps);
  const TG* gp = gate + t * g_stride + (long long)h * P;
  T* dst = out + t * out_stride + (long long)h * P;
  for (int e = lane; e < P; e += 32) {
    const float g = to_f(gp[e]);
    dst[e] = from_f<T>(op[e] * rstd * (g / (1.0f + expf(-g))));
  }
}
}  // namespace

// rot = 0: nothing is rotated (inv_freq may then be null).  dtype: the projection's type.
FMX_EXPORT int fmx_retention_prepare(const void* proj, long long stride, int dtype, const int* positions, const float* inv_freq,
                                     const float* decay, float* out_xbc, float* out_dd, int T, int H, int D, int P, int rot,
                                     float k_scale, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || H <= 0 || D <= 0 || P <= 0 || rot < 0 || rot > D || (rot & 1))
    return fmx_fail("fmx_retention_prepare: bad sizes T=%d H=%d D=%d P=%d rot=%d", T, H, D, P, rot);
  if (rot > 0 && inv_freq == nullptr) return fmx_fail("fmx_retention_prepare: rot=%d needs a frequency table", rot);
  if (stride < 2LL * H * D + (long long)H * P) return fmx_fail("fmx_retention_prepare: rows too narrow");
  const size_t smem = (size_t)rot * sizeof(float);
  if (dtype == FMX_F32)
    fmx_launch(retention_prepare_kernel<float>, dim3(T), dim3(128), smem, stream, (const float*)proj, stride, positions, inv_freq,
               decay, out_xbc, out_dd, H, D, P, rot, k_scale);
  else if (dtype == FMX_BF16)
    fmx_launch(retention_prepare_kernel<bf16>, dim3(T), dim3(128), smem, stream, (const bf16*)proj, stride, positions, inv_freq,
               decay, out_xbc, out_dd, H, D, P, rot, k_scale);
  else
    return fmx_fail("fmx_retention_prepare: unknown dtype %d", dtype);
  FMX_LAUNCH_CHECK();
  return 0;
}

// o [T, H*P] 32-bit; gate rows of g_stride elements of type g_dtype; out rows of out_stride elements of type dtype.
FMX_EXPORT int fmx_retention_gate_norm(const float* o, const void* gate, long long g_stride, int g_dtype, void* out,
                                       long long out_stride, int dtype, int T, int H, int P, float eps, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || H <= 0 || P <= 0 || g_stride < (long long)H * P || out_stride < (long long)H * P)
    return fmx_fail("fmx_retention_gate_norm: bad sizes T=%d H=%d P=%d", T, H, P);
  const long long n = (long long)T * H, grid = (n + 3) / 4;
  if (grid > 2147483647LL) return fmx_fail("fmx_retention_gate_norm: batch too large");
#define FMX_RGN(TG, TO)                                                                                               \
  fmx_launch(retention_gate_norm_kernel<TG, TO>, dim3((unsigned)grid), dim3(128), 0, stream, o, (const TG*)gate, g_stride, \
             (TO*)out, out_stride, n, H, P, eps)
  if (g_dtype == FMX_F32 && dtype == FMX_F32) FMX_RGN(float, float);
  else if (g_dtype == FMX_F32 && dtype == FMX_BF16) FMX_RGN(float, bf16);
  else if (g_dtype == FMX_BF16 && dtype == FMX_BF16) FMX_RGN(bf16, bf16);
  else return fmx_fail("fmx_retention_gate_norm: unknown dtypes %d, %d", g_dtype, dtype);
#undef FMX_RGN
  FMX_LAUNCH_CHECK();
  return 0;
}
