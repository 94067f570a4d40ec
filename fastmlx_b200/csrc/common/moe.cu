// A routed feed-forward's own kernels: the router's choice and the experts' activation.
//
// moe_route: one warp per token.  Scores s = softmax(z) over all E experts (32-bit).  With groups (E / groups
// neighbouring experts each), a group scores as its best member and only the `keep` best groups may be chosen from.
// The `top` best allowed experts are chosen (the lower index on a tie); the token's weights are their scores as they
// are, not renormalised.  Out: a dense row of weights [E], zero where an expert is not chosen, and the chosen
// indices [top] in the order of choice.
//
// moe_expert_act: the hidden layer of all experts side by side.  gu[t] holds F gate values and then F up values,
// F = E * ff (+ ff_shared for an expert that every token uses); y = w * g' sigmoid(1.702 g') (u' + 1) with
// g' = min(g, limit), u' = clamp(u, -limit, limit), and w the token's weight for the column's expert (1 for the
// shared one).  A column whose expert the token did not choose is zero, so that one product with all the experts'
// down matrices side by side gives the weighted sum.
#include <math.h>
#include "common.cuh"

namespace {
constexpr int ROUTE_WARPS = 4;

__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, i, o);
    if (ov > v || (ov == v && oi < i)) { v = ov; i = oi; }
  }
}

__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const float* z, long long z_stride, int T, int E, int top, int groups, int keep, float* weights,
                 int* chosen, const float* __restrict__ choice_bias, float weight_scale) {
  extern __shared__ float smem[];               // per warp: E scores, E marks (as floats), `groups` group scores
  pdl_wait();
  pdl_trigger();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= T) return;
  float* s = smem + (size_t)warp * (2 * E + groups);
  float* ok = s + E;                            // 1: may be chosen, 0: not (group not kept, or chosen already)
  float* gs = ok + E;
  const float* zr = z + (long long)t * z_stride;
  float m = -INFINITY;
  for (int e = lane; e < E; e += 32) m = fmaxf(m, zr[e]);
  m = warp_max(m);
  float sum = 0.f;
  for (int e = lane; e < E; e += 32) {
    const float p = expf(zr[e] - m);
    s[e] = p;
    sum += p;
  }
  sum = warp_sum(sum);
  const float inv = 1.0f / sum;
  for (int e = lane; e < E; e += 32) {
    s[e] *= inv;
    ok[e] = 1.f;
    weights[(long long)t * E + e] = 0.f;
  }
  __syncwarp();
  if (groups > 1 && keep < groups) {
    const int per = E / groups;
    for (int g = lane; g < groups; g += 32) {
      float best = -1.f;
      for (int e = g * per; e < (g + 1) * per; ++e) best = fmaxf(best, s[e]);
      gs[g] = best;
    }
    for (int e = lane; e < E; e += 32) ok[e] = 0.f;
    __syncwarp();
    for (int k = 0; k < keep; ++k) {
      float bv = -2.f;
      int bi = 0x7fffffff;
      for (int g = lane; g < groups; g += 32)
        if (gs[g] > bv) { bv = gs[g]; bi = g; }
      warp_argmax(bv, bi);
      if (bi >= groups) break;
      for (int e = bi * per + lane; e < (bi + 1) * per; e += 32) ok[e] = 1.f;
      if (lane == 0) gs[bi] = -3.f;
      __syncwarp();
    }
  }
  for (int k = 0; k < top; ++k) {
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float cv = s[e] + (choice_bias != nullptr ? choice_bias[e] : 0.f);    // chosen by score + bias, weighed by score
      if (ok[e] != 0.f && (cv > bv || bi == 0x7fffffff)) { bv = cv; bi = e; }
    }
    warp_argmax(bv, bi);
    if (bi >= E) {                               // fewer allowed experts than `top`
      if (lane == 0 && chosen != nullptr) chosen[(long long)t * top + k] = -1;
      continue;
    }
    if (lane == 0) {
      ok[bi] = 0.f;
      weights[(long long)t * E + bi] = s[bi] * weight_scale;
      if (chosen != nullptr) chosen[(long long)t * top + k] = bi;
    }
    __syncwarp();
  }
}

template <typename T>
__global__ void moe_expert_act_kernel(const T* gu, long long gu_stride, const float* weights, T* out, long long out_stride,
                                      long long rows, int E, int ff, int F, float limit, float limit_shared, int block) {
  pdl_wait();
  pdl_trigger();
  const long long n = rows * F;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / F;
    const int c = (int)(idx - r * F);
    const int e = c / ff;
    const float w = e < E ? weights[r * E + e] : 1.0f;
    float y = 0.f;
    if (w != 0.f) {
      const float lim = e < E ? limit : limit_shared;
      // block > 0: gate and up values alternate in blocks of `block`; else F gates, then F ups
      const long long gi = block > 0 ? (long long)(c / block) * 2 * block + c % block : c;
      const long long ui = block > 0 ? gi + block : (long long)F + c;
      const float g = fminf(to_f(gu[r * gu_stride + gi]), lim);
      const float u = fminf(fmaxf(to_f(gu[r * gu_stride + ui]), -lim), lim);
      y = w * (g / (1.0f + expf(-1.702f * g))) * (u + 1.0f);
    }
    out[r * out_stride + c] = from_f<T>(y);
  }
}
// The same for bfloat16 rows in 16-byte pieces (eight columns of one expert: ff is a multiple of 8).
__global__ void moe_expert_act_vec_kernel(const bf16* gu, long long gu_stride, const float* weights, bf16* out, long long out_stride,
                                          long long rows, int E, int ff, int F, float limit, float limit_shared, int block) {
  pdl_wait();
  pdl_trigger();
  const int f8 = F / 8;
  const long long n = rows * f8;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / f8;
    const int c = (int)(idx - r * f8) * 8;
    const int e = c / ff;
    const float w = e < E ? weights[r * E + e] : 1.0f;
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if (w != 0.f) {
      const float lim = e < E ? limit : limit_shared;
      const long long gi = block > 0 ? (long long)(c / block) * 2 * block + c % block : c;
      const long long ui = block > 0 ? gi + block : (long long)F + c;
      const uint4 g4 = *reinterpret_cast<const uint4*>(gu + r * gu_stride + gi);
      const uint4 u4 = *reinterpret_cast<const uint4*>(gu + r * gu_stride + ui);
      const __nv_bfloat162* gp = reinterpret_cast<const __nv_bfloat162*>(&g4);
      const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u4);
      __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 g = __bfloat1622float2(gp[i]), u = __bfloat1622float2(up[i]);
        const float g0 = fminf(g.x, lim), g1 = fminf(g.y, lim);
        const float u0 = fminf(fmaxf(u.x, -lim), lim), u1 = fminf(fmaxf(u.y, -lim), lim);
        op[i] = __floats2bfloat162_rn(w * (g0 / (1.0f + expf(-1.702f * g0))) * (u0 + 1.0f),
                                      w * (g1 / (1.0f + expf(-1.702f * g1))) * (u1 + 1.0f));
      }
    }
    *reinterpret_cast<uint4*>(out + r * out_stride + c) = o;
  }
}

// Experts without a gate, side by side: u[t] holds F = E * ff (+ a shared expert's) hidden values; y = w * act(u) with w
// the token's weight for the column's expert, zero where it did not choose it.  The shared columns at the end weigh
// sigmoid(shared_gate[t]) where a gate is given, else 1.  act: 0 relu^2, 1 gelu (tanh form), 2 silu.
template <typename T>
__global__ void moe_plain_act_kernel(const T* u, long long u_stride, const float* weights, const float* shared_gate,
                                     long long sg_stride, T* out, long long out_stride, long long rows, int E, int ff, int F,
                                     int act) {
  pdl_wait();
  pdl_trigger();
  const long long n = rows * F;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / F;
    const int c = (int)(idx - r * F);
    const int e = c / ff;
    float w;
    if (e < E) w = weights[r * E + e];
    else w = shared_gate != nullptr ? 1.0f / (1.0f + expf(-shared_gate[r * sg_stride])) : 1.0f;
    float y = 0.f;
    if (w != 0.f) {
      const float x = to_f(u[r * u_stride + c]);
      float a;
      if (act == 0) { const float p = fmaxf(x, 0.f); a = p * p; }
      else if (act == 1) a = 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
      else a = x / (1.0f + expf(-x));
      y = w * a;
    }
    out[r * out_stride + c] = from_f<T>(y);
  }
}
}  // namespace

// choice_bias ([E], may be null): added to the scores for the choice only; weight_scale multiplies the chosen scores.
FMX_EXPORT int fmx_moe_route_biased(const float* z, long long z_stride, int T, int E, int top, int groups, int keep,
                                    float* weights, int* chosen, const float* choice_bias, float weight_scale,
                                    cudaStream_t stream);
FMX_EXPORT int fmx_moe_route(const float* z, long long z_stride, int T, int E, int top, int groups, int keep, float* weights,
                             int* chosen, cudaStream_t stream) {
  return fmx_moe_route_biased(z, z_stride, T, E, top, groups, keep, weights, chosen, nullptr, 1.0f, stream);
}

FMX_EXPORT int fmx_moe_route_biased(const float* z, long long z_stride, int T, int E, int top, int groups, int keep,
                                    float* weights, int* chosen, const float* choice_bias, float weight_scale,
                                    cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || E <= 0 || top <= 0 || top > E || groups <= 0 || E % groups || keep <= 0 || z_stride < E)
    return fmx_fail("fmx_moe_route: bad sizes T=%d E=%d top=%d groups=%d keep=%d", T, E, top, groups, keep);
  const size_t smem = (size_t)ROUTE_WARPS * (2 * (size_t)E + groups) * sizeof(float);
  if (smem > 48 * 1024) return fmx_fail("fmx_moe_route: %d experts are more than the kernel's shared memory holds", E);
  fmx_launch(moe_route_kernel, dim3((T + ROUTE_WARPS - 1) / ROUTE_WARPS), dim3(ROUTE_WARPS * 32), smem, stream, z, z_stride, T, E,
             top, groups, keep, weights, chosen, choice_bias, weight_scale);
  FMX_LAUNCH_CHECK();
  return 0;
}

// ff_shared = F - E * ff columns at the end belong to an expert that every token uses with weight 1.
// gu_block > 0 (a multiple of 8 that divides F): gate and up values alternate in blocks of that many instead of F gates, then F ups.
FMX_EXPORT int fmx_moe_expert_act(const void* gu, long long gu_stride, const float* weights, void* out, long long out_stride,
                                  int rows, int E, int ff, int F, float limit, float limit_shared, int dtype, int gu_block,
                                  cudaStream_t stream) {
  if (gu_block < 0 || (gu_block > 0 && (F % gu_block || gu_block % 8))) return fmx_fail("fmx_moe_expert_act: blocks of %d do not fit %d columns", gu_block, F);
  if (rows == 0 || F == 0) return 0;
  if (rows < 0 || E < 0 || ff <= 0 || F < E * ff || gu_stride < 2LL * F || out_stride < F)
    return fmx_fail("fmx_moe_expert_act: bad sizes rows=%d E=%d ff=%d F=%d", rows, E, ff, F);
  const bool vec = dtype == FMX_BF16 && F % 8 == 0 && ff % 8 == 0 && (E * ff) % 8 == 0 && gu_stride % 8 == 0 && out_stride % 8 == 0 &&
                   ((uintptr_t)gu & 15) == 0 && ((uintptr_t)out & 15) == 0;
  const long long n = (long long)rows * (vec ? F / 8 : F), cap = (long long)fmx_num_sms() * 16;
  const int block = 256;
  const int grid = (int)((n + block - 1) / block < cap ? (n + block - 1) / block : cap);
  if (vec)
    fmx_launch(moe_expert_act_vec_kernel, dim3(grid), dim3(block), 0, stream, (const bf16*)gu, gu_stride, weights, (bf16*)out,
               out_stride, (long long)rows, E, ff, F, limit, limit_shared, gu_block);
  else if (dtype == FMX_F32)
    fmx_launch(moe_expert_act_kernel<float>, dim3(grid), dim3(block), 0, stream, (const float*)gu, gu_stride, weights, (float*)out,
               out_stride, (long long)rows, E, ff, F, limit, limit_shared, gu_block);
  else if (dtype == FMX_BF16)
    fmx_launch(moe_expert_act_kernel<bf16>, dim3(grid), dim3(block), 0, stream, (const bf16*)gu, gu_stride, weights, (bf16*)out,
               out_stride, (long long)rows, E, ff, F, limit, limit_shared, gu_block);
  else
    return fmx_fail("fmx_moe_expert_act: unknown dtype %d", dtype);
  FMX_LAUNCH_CHECK();
  return 0;
}

namespace {
// moe_plain_act for bfloat16 rows in 16-byte pieces (eight columns of one expert: ff and the experts' columns are multiples of 8).
__global__ void moe_plain_act_vec_kernel(const bf16* u, long long u_stride, const float* weights, const float* shared_gate,
                                         long long sg_stride, bf16* out, long long out_stride, long long rows, int E, int ff,
                                         int F, int act) {
  pdl_wait();
  pdl_trigger();
  const int f8 = F / 8;
  const long long n = rows * f8;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / f8;
    const int c = (int)(idx - r * f8) * 8;
    const int e = c / ff;
    float w;
    if (e < E) w = weights[r * E + e];
    else w = shared_gate != nullptr ? 1.0f / (1.0f + expf(-shared_gate[r * sg_stride])) : 1.0f;
    uint4 o = make_uint4(0u, 0u, 0u, 0u);
    if (w != 0.f) {
      const uint4 u4 = *reinterpret_cast<const uint4*>(u + r * u_stride + c);
      const __nv_bfloat162* up = reinterpret_cast<const __nv_bfloat162*>(&u4);
      __nv_bfloat162* op = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float2 x = __bfloat1622float2(up[i]);
        float a0, a1;
        if (act == 0) { const float p0 = fmaxf(x.x, 0.f), p1 = fmaxf(x.y, 0.f); a0 = p0 * p0; a1 = p1 * p1; }
        else if (act == 1) {
          a0 = 0.5f * x.x * (1.0f + tanhf(0.7978845608028654f * (x.x + 0.044715f * x.x * x.x * x.x)));
          a1 = 0.5f * x.y * (1.0f + tanhf(0.7978845608028654f * (x.y + 0.044715f * x.y * x.y * x.y)));
        } else { a0 = x.x / (1.0f + expf(-x.x)); a1 = x.y / (1.0f + expf(-x.y)); }
        op[i] = __floats2bfloat162_rn(w * a0, w * a1);
      }
    }
    *reinterpret_cast<uint4*>(out + r * out_stride + c) = o;
  }
}
}  // namespace

FMX_EXPORT int fmx_moe_plain_act(const void* u, long long u_stride, const float* weights, const float* shared_gate,
                                 long long sg_stride, void* out, long long out_stride, int rows, int E, int ff, int F, int act,
                                 int dtype, cudaStream_t stream) {
  if (rows == 0 || F == 0) return 0;
  if (rows < 0 || E < 0 || ff <= 0 || F < E * ff || u_stride < F || out_stride < F || act < 0 || act > 2)
    return fmx_fail("fmx_moe_plain_act: bad sizes rows=%d E=%d ff=%d F=%d act=%d", rows, E, ff, F, act);
  const bool vec = dtype == FMX_BF16 && F % 8 == 0 && ff % 8 == 0 && (E * ff) % 8 == 0 && u_stride % 8 == 0 && out_stride % 8 == 0 &&
                   ((uintptr_t)u & 15) == 0 && ((uintptr_t)out & 15) == 0;
  const long long n = (long long)rows * (vec ? F / 8 : F), cap = (long long)fmx_num_sms() * 16;
  const int block = 256;
  const int grid = (int)((n + block - 1) / block < cap ? (n + block - 1) / block : cap);
  if (vec)
    fmx_launch(moe_plain_act_vec_kernel, dim3(grid), dim3(block), 0, stream, (const bf16*)u, u_stride, weights, shared_gate, sg_stride,
               (bf16*)out, out_stride, (long long)rows, E, ff, F, act);
  else if (dtype == FMX_F32)
    fmx_launch(moe_plain_act_kernel<float>, dim3(grid), dim3(block), 0, stream, (const float*)u, u_stride, weights, shared_gate,
               sg_stride, (float*)out, out_stride, (long long)rows, E, ff, F, act);
  else if (dtype == FMX_BF16)
    fmx_launch(moe_plain_act_kernel<bf16>, dim3(grid), dim3(block), 0, stream, (const bf16*)u, u_stride, weights, shared_gate,
               sg_stride, (bf16*)out, out_stride, (long long)rows, E, ff, F, act);
  else
    return fmx_fail("fmx_moe_plain_act: unknown dtype %d", dtype);
  FMX_LAUNCH_CHECK();
  return 0;
}
