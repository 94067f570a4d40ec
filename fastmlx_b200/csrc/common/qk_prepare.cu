// Queries and keys made ready for attention in one pass: rotary positions on the first `rot`
// dimensions of every head, then (optionally) each head divided by its root mean square, then
// the keys and values written into the layer's pages.  With `norm_first` the order is the other
// one: a head is divided by its root mean square (and multiplied by a weight of hd values, one for
// the queries and one for the keys, shared by their heads) and rotated after that.
//
// qkv is [T, nh*hd + nkv*hd + nkv*vd] as the projection left it, of its own type (a product that
// leaves in 32-bit feeds a bfloat16 cache); `bias`, if given, is added here, in 32-bit.  The queries
// leave in 32-bit, [T, nh*hd]: scores are then taken from unrounded queries.  Keys and values go
// to slot_mapping[t] of a cache whose pages hold [nkv, page_size, hd] keys followed by
// [nkv, page_size, vd] values.  Angles (position * inv_freq[j]), sines, cosines, the sum of
// squares and the division are 32-bit; the sum of squares of a head is taken in an order that
// depends on the head size alone.
#include "common.cuh"

namespace {
constexpr int QKP_WARPS = 4;

template <typename TI, typename T>
__global__ void __launch_bounds__(QKP_WARPS * 32)
qk_prepare_kernel(const TI* qkv, long long row_stride, const int* positions, const float* __restrict__ inv_freq,
                  const long long* slot_mapping, float* q_out, T* kv, int nh, int nkv, int hd, int vd, int rot,
                  int interleaved, float norm_eps, int page_size, long long num_pages, int* status,
                  const float* __restrict__ bias, const float* __restrict__ q_weight, const float* __restrict__ k_weight,
                  int norm_first) {
  extern __shared__ float smem[];               // [rot/2] sines, [rot/2] cosines, then a head per warp
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = rot / 2;
  float* sn = smem;
  float* cs = smem + half;
  float* buf = smem + rot + warp * hd;
  const TI* row = qkv + (long long)t * row_stride;
  const float pos = (float)positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &sn[j], &cs[j]);
  long long slot = (kv != nullptr && slot_mapping != nullptr) ? slot_mapping[t] : -1;
  if (slot >= num_pages * page_size) {
    if (threadIdx.x == 0) fmx_set_status(status, FMX_BAD_SLOT, slot, t);
    slot = -1;
  }
  const long long page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? (int)(slot - page * page_size) : 0;
  const long long page_elems = (long long)nkv * page_size * (hd + vd);
  __syncthreads();
  for (int h = warp; h < nh + nkv; h += QKP_WARPS) {
    const TI* src = row + (long long)h * hd;
    const float* hw = h < nh ? q_weight : k_weight;
    float ss0 = 0.f;
    for (int e = lane; e < hd; e += 32) {
      const float v = to_f(src[e]) + (bias != nullptr ? bias[(long long)h * hd + e] : 0.f);
      buf[e] = v;
      ss0 = fmaf(v, v, ss0);
    }
    if (norm_first && norm_eps >= 0.f) {
      const float m0 = 1.0f / sqrtf(warp_sum(ss0) / (float)hd + norm_eps);
      for (int e = lane; e < hd; e += 32) buf[e] = buf[e] * m0 * (hw != nullptr ? hw[e] : 1.0f);
    }
    __syncwarp();
    float ss = 0.f;
    float val[8];                               // head sizes up to 256
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int e = lane + 32 * i;
      float v = 0.f;
      if (e < hd) {
        v = buf[e];
        if (e < rot) {
          int j, other;
          bool first;
          if (interleaved) { j = e >> 1; first = (e & 1) == 0; other = first ? e + 1 : e - 1; }
          else { first = e < half; j = first ? e : e - half; other = first ? e + half : e - half; }
          float x, y;
          if (first) rope_pair(v, buf[other], sn[j], cs[j], x, y);
          else rope_pair(buf[other], v, sn[j], cs[j], y, x);      // x: this element's new value in either case
          v = x;
        }
        ss = fmaf(v, v, ss);
      }
      val[i] = v;
    }
    float mul = 1.0f;
    if (!norm_first && norm_eps >= 0.f) {
      mul = 1.0f / sqrtf(warp_sum(ss) / (float)hd + norm_eps);
      if (hw != nullptr) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int e = lane + 32 * i;
          if (e < hd) val[i] *= hw[e];
        }
      }
    }
    if (h < nh) {
      float* dst = q_out + ((long long)t * nh + h) * hd;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        if (e < hd) dst[e] = val[i] * mul;
      }
    } else if (slot >= 0) {
      T* dst = kv + page * page_elems + ((long long)(h - nh) * page_size + off) * hd;
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const int e = lane + 32 * i;
        if (e < hd) dst[e] = from_f<T>(val[i] * mul);
      }
    }
    __syncwarp();
  }
  if (slot < 0) return;
  const TI* vsrc = row + (long long)(nh + nkv) * hd;
  const float* vbias = bias != nullptr ? bias + (long long)(nh + nkv) * hd : nullptr;
  T* vdst = kv + page * page_elems + (long long)nkv * page_size * hd;
  for (int it = threadIdx.x; it < nkv * vd; it += blockDim.x) {
    const int g = it / vd, e = it - g * vd;
    vdst[((long long)g * page_size + off) * vd + e] = from_f<T>(to_f(vsrc[it]) + (vbias != nullptr ? vbias[it] : 0.f));
  }
}

// The form that normalises q and k over the whole projection: all nh * hd query values of a token are divided by
// their common root mean square and multiplied by a weight of that width (the keys' nkv * hd values likewise), before
// the rotation.  With `values_from_keys` the row holds no values: a token's values are its keys as projected, before
// norm and rotation (vd = hd).  One block per token; the two sums of squares are taken by the whole block in an
// order that depends on the sizes alone.
template <typename TI, typename T>
__global__ void __launch_bounds__(QKP_WARPS * 32)
qk_prepare_whole_kernel(const TI* qkv, long long row_stride, const int* positions, const float* __restrict__ inv_freq,
                        const long long* slot_mapping, float* q_out, T* kv, int nh, int nkv, int hd, int vd, int rot,
                        int interleaved, float norm_eps, int page_size, long long num_pages, int* status,
                        const float* __restrict__ bias, const float* __restrict__ q_weight,
                        const float* __restrict__ k_weight, int values_from_keys) {
  extern __shared__ float smem[];               // [rot/2] sines, [rot/2] cosines, then a head per warp
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = rot / 2;
  float* sn = smem;
  float* cs = smem + half;
  float* buf = smem + rot + warp * hd;
  const TI* row = qkv + (long long)t * row_stride;
  const float pos = (float)positions[t];
  for (int j = threadIdx.x; j < half; j += blockDim.x) sincosf(pos * inv_freq[j], &sn[j], &cs[j]);
  long long slot = (kv != nullptr && slot_mapping != nullptr) ? slot_mapping[t] : -1;
  if (slot >= num_pages * page_size) {
    if (threadIdx.x == 0) fmx_set_status(status, FMX_BAD_SLOT, slot, t);
    slot = -1;
  }
  const long long page = slot >= 0 ? slot / page_size : 0;
  const int off = slot >= 0 ? (int)(slot - page * page_size) : 0;
  const long long page_elems = (long long)nkv * page_size * (hd + vd);
  const int nq = nh * hd, nk = nkv * hd;
  float sq = 0.f, sk = 0.f;
  for (int e = threadIdx.x; e < nq; e += blockDim.x) {
    const float v = to_f(row[e]) + (bias != nullptr ? bias[e] : 0.f);
    sq = fmaf(v, v, sq);
  }
  for (int e = threadIdx.x; e < nk; e += blockDim.x) {
    const float v = to_f(row[nq + e]) + (bias != nullptr ? bias[nq + e] : 0.f);
    sk = fmaf(v, v, sk);
  }
  sq = block_sum<QKP_WARPS * 32>(sq);
  sk = block_sum<QKP_WARPS * 32>(sk);           // (its barriers also publish the sines and cosines)
  const bool normed = norm_eps >= 0.f;
  const float mq = normed ? 1.0f / sqrtf(sq / (float)nq + norm_eps) : 1.0f;
  const float mk = (normed && nk > 0) ? 1.0f / sqrtf(sk / (float)nk + norm_eps) : 1.0f;
  for (int h = warp; h < nh + nkv; h += QKP_WARPS) {
    const TI* src = row + (long long)h * hd;
    const float* hw = h < nh ? (q_weight != nullptr ? q_weight + (long long)h * hd : nullptr)
                             : (k_weight != nullptr ? k_weight + (long long)(h - nh) * hd : nullptr);
    const float mul = h < nh ? mq : mk;
    T* vdst = (h >= nh && slot >= 0 && values_from_keys)
                  ? kv + page * page_elems + (long long)nkv * page_size * hd + ((long long)(h - nh) * page_size + off) * vd
                  : nullptr;
    for (int e = lane; e < hd; e += 32) {
      const float v = to_f(src[e]) + (bias != nullptr ? bias[(long long)h * hd + e] : 0.f);
      if (vdst != nullptr) vdst[e] = from_f<T>(v);                 // the value: the key as it was projected
      buf[e] = v * mul * (hw != nullptr ? hw[e] : 1.0f);
    }
    __syncwarp();
    T* kdst = (h >= nh && slot >= 0) ? kv + page * page_elems + ((long long)(h - nh) * page_size + off) * hd : nullptr;
    float* qdst = h < nh ? q_out + ((long long)t * nh + h) * hd : nullptr;
    for (int e = lane; e < hd; e += 32) {
      float v = buf[e];
      if (e < rot) {
        int j, other;
        bool first;
        if (interleaved) { j = e >> 1; first = (e & 1) == 0; other = first ? e + 1 : e - 1; }
        else { first = e < half; j = first ? e : e - half; other = first ? e + half : e - half; }
        float x, y;
        if (first) rope_pair(v, buf[other], sn[j], cs[j], x, y);
        else rope_pair(buf[other], v, sn[j], cs[j], y, x);          // x: this element's new value in either case
        v = x;
      }
      if (qdst != nullptr) qdst[e] = v;
      else if (kdst != nullptr) kdst[e] = from_f<T>(v);
    }
    __syncwarp();
  }
  if (slot < 0 || values_from_keys) return;
  const TI* vsrc = row + (long long)(nh + nkv) * hd;
  const float* vbias = bias != nullptr ? bias + (long long)(nh + nkv) * hd : nullptr;
  T* vdst = kv + page * page_elems + (long long)nkv * page_size * hd;
  for (int it = threadIdx.x; it < nkv * vd; it += blockDim.x) {
    const int g = it / vd, e = it - g * vd;
    vdst[((long long)g * page_size + off) * vd + e] = from_f<T>(to_f(vsrc[it]) + (vbias != nullptr ? vbias[it] : 0.f));
  }
}
}  // namespace

// rot = 0: nothing is rotated; norm_eps < 0: heads are not normalised; kv or slot_mapping null:
// nothing is stored (a layer that reads another's cache then passes nkv = 0 as well).  in_dtype: the
// type of qkv; dtype: the cache's.  bias (the whole row's, 32-bit), q_weight, k_weight may be null.
FMX_EXPORT int fmx_qk_prepare_ex(const void* qkv, long long row_stride, const int* positions, const float* inv_freq,
                                 const long long* slot_mapping, float* q_out, void* kv, int T, int nh, int nkv, int hd,
                                 int vd, int rot, int interleaved, float norm_eps, int page_size, long long num_pages,
                                 int in_dtype, int dtype, const float* bias, const float* q_weight, const float* k_weight,
                                 int norm_first, int* status, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || nh < 0 || nkv < 0 || hd <= 0 || vd <= 0 || hd > 256 || rot < 0 || rot > hd || (rot & 1) || page_size <= 0)
    return fmx_fail("fmx_qk_prepare: bad sizes T=%d nh=%d nkv=%d hd=%d vd=%d rot=%d", T, nh, nkv, hd, vd, rot);
  if (rot > 0 && inv_freq == nullptr) return fmx_fail("fmx_qk_prepare: rot=%d needs a frequency table", rot);
  if (row_stride < (long long)(nh + nkv) * hd + (long long)nkv * vd) return fmx_fail("fmx_qk_prepare: row stride too small");
  const size_t smem = ((size_t)rot + (size_t)QKP_WARPS * hd) * sizeof(float);
#define FMX_QKP(TI, TKV)                                                                                                  \
  fmx_launch(qk_prepare_kernel<TI, TKV>, dim3(T), dim3(QKP_WARPS * 32), smem, stream, (const TI*)qkv, row_stride, positions, \
             inv_freq, slot_mapping, q_out, (TKV*)kv, nh, nkv, hd, vd, rot, interleaved, norm_eps, page_size, num_pages,  \
             status, bias, q_weight, k_weight, norm_first)
  if (in_dtype == FMX_F32 && dtype == FMX_F32)
    FMX_QKP(float, float);
  else if (in_dtype == FMX_BF16 && dtype == FMX_BF16)
    FMX_QKP(bf16, bf16);
  else if (in_dtype == FMX_F32 && dtype == FMX_BF16)
    FMX_QKP(float, bf16);
  else
    return fmx_fail("fmx_qk_prepare: no kernel for an input of type %d and a cache of type %d", in_dtype, dtype);
#undef FMX_QKP
  FMX_LAUNCH_CHECK();
  return 0;
}

FMX_EXPORT int fmx_qk_prepare(const void* qkv, long long row_stride, const int* positions, const float* inv_freq,
                              const long long* slot_mapping, float* q_out, void* kv, int T, int nh, int nkv, int hd, int vd,
                              int rot, int interleaved, float norm_eps, int page_size, long long num_pages, int dtype,
                              int* status, cudaStream_t stream) {
  return fmx_qk_prepare_ex(qkv, row_stride, positions, inv_freq, slot_mapping, q_out, kv, T, nh, nkv, hd, vd, rot, interleaved,
                           norm_eps, page_size, num_pages, dtype, dtype, nullptr, nullptr, nullptr, 0, status, stream);
}

// q and k normalised over the whole projection, before the rotation (q_weight [nh*hd], k_weight [nkv*hd], either may be
// null); values_from_keys: the row holds q | k only and a token's values are its keys as projected (vd = hd).
FMX_EXPORT int fmx_qk_prepare_whole(const void* qkv, long long row_stride, const int* positions, const float* inv_freq,
                                    const long long* slot_mapping, float* q_out, void* kv, int T, int nh, int nkv, int hd,
                                    int vd, int rot, int interleaved, float norm_eps, int page_size, long long num_pages,
                                    int in_dtype, int dtype, const float* bias, const float* q_weight, const float* k_weight,
                                    int values_from_keys, int* status, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || nh < 0 || nkv < 0 || hd <= 0 || vd <= 0 || hd > 256 || rot < 0 || rot > hd || (rot & 1) || page_size <= 0)
    return fmx_fail("fmx_qk_prepare_whole: bad sizes T=%d nh=%d nkv=%d hd=%d vd=%d rot=%d", T, nh, nkv, hd, vd, rot);
  if (values_from_keys && vd != hd) return fmx_fail("fmx_qk_prepare_whole: values that are the keys have the keys' width");
  if (rot > 0 && inv_freq == nullptr) return fmx_fail("fmx_qk_prepare_whole: rot=%d needs a frequency table", rot);
  if (row_stride < (long long)(nh + nkv) * hd + (values_from_keys ? 0 : (long long)nkv * vd))
    return fmx_fail("fmx_qk_prepare_whole: row stride too small");
  const size_t smem = ((size_t)rot + (size_t)QKP_WARPS * hd) * sizeof(float);
#define FMX_QKW(TI, TKV)                                                                                                 \
  fmx_launch(qk_prepare_whole_kernel<TI, TKV>, dim3(T), dim3(QKP_WARPS * 32), smem, stream, (const TI*)qkv, row_stride,  \
             positions, inv_freq, slot_mapping, q_out, (TKV*)kv, nh, nkv, hd, vd, rot, interleaved, norm_eps, page_size, \
             num_pages, status, bias, q_weight, k_weight, values_from_keys)
  if (in_dtype == FMX_F32 && dtype == FMX_F32)
    FMX_QKW(float, float);
  else if (in_dtype == FMX_BF16 && dtype == FMX_BF16)
    FMX_QKW(bf16, bf16);
  else if (in_dtype == FMX_F32 && dtype == FMX_BF16)
    FMX_QKW(float, bf16);
  else
    return fmx_fail("fmx_qk_prepare_whole: no kernel for an input of type %d and a cache of type %d", in_dtype, dtype);
#undef FMX_QKW
  FMX_LAUNCH_CHECK();
  return 0;
}
