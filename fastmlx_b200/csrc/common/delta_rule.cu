// The gated delta rule: a linear-attention mixer whose per-request state is a matrix per head.
//
// Per head, with key k, query q (size D), value v (size Dv), decay g in (0, 1) and write strength
// beta in (0, 1), a token does, in this order,
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q,
// so the read-out sees the token's own write.  S [D, Dv] lives in 32-bit in a state slot of the
// request and is carried from step to step; so are the last taps-1 inputs of the short causal
// convolutions that q, k and v pass through.
//
// Four kernels:
//   delta_prepare     per token: convolution + SiLU of the projected q | k | v channels (inputs before the
//                     portion's start come from the slot's convolution state), q and k made unit vectors per head
//                     (q also times D^-1/2), beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias)).
//   conv_state_update per request: the last taps-1 inputs of the portion replace the convolution state.
//   delta_rule        the recurrence.  Columns of S are independent (column j needs v_j only), so a column is
//                     given to 8 to 32 adjacent lanes that hold 8 of its values each in registers; the
//                     tokens of a request's portion are walked in order, their operands staged through shared
//                     memory a run of tokens ahead.
//   gated_rmsnorm     o of each head divided by its root mean square, times a weight, times SiLU(gate).
//
// A slot's state is one run of 32-bit floats: S^T of every head, [H, Dv, D], and then the convolution inputs,
// [taps-1, C].  Everything is 32-bit but the projections that come in and the activations that go out.  No sum's
// order depends on how a request's tokens were cut into steps or on what else is in the batch.
#include <math.h>
#include "common.cuh"

#include "conv_state.cuh"

namespace {

// proj [T, stride]: q (G*D) | k (G*D) | v (H*Dv) | ... ; ab [T, ab_stride] 32-bit: b (H) | a (H).
// out_qkv [T, C] 32-bit; out_gb [T, 2H]: decay | beta.
template <typename T>
__global__ void __launch_bounds__(128)
delta_prepare_kernel(const T* proj, long long stride, const float* ab, long long ab_stride,
                     const float* __restrict__ conv_w, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                     const int* token_row, const int* row_start, const int* row_slot, const float* state,
                     long long slot_stride, long long conv_off, float* out_qkv, float* out_gb, int H, int G, int D,
                     int Dv, int taps, int R, int max_slots, int* status) {
  extern __shared__ float vals[];               // the token's C channels after convolution and SiLU
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const int C = 2 * G * D + H * Dv;
  const int r = token_row[t];
  float* oq = out_qkv + (long long)t * C;
  float* og = out_gb + (long long)t * 2 * H;
  const int slot = (r >= 0 && r < R) ? row_slot[r] : -1;
  if (slot < 0 || slot >= max_slots) {          // a padding row of a captured step, or a bad row: nothing to do
    if (r < 0 || r >= R) { if (threadIdx.x == 0) fmx_set_status(status, FMX_BAD_ROW, r, t); }
    else if (slot >= max_slots && threadIdx.x == 0) fmx_set_status(status, FMX_BAD_SLOT, slot, t);
    for (int c = threadIdx.x; c < C; c += blockDim.x) oq[c] = 0.f;
    for (int c = threadIdx.x; c < 2 * H; c += blockDim.x) og[c] = 0.f;
    return;
  }
  const int first = row_start[r];
  const int i = t - first;                       // the token's place in its portion
  const float* cstate = state + (long long)slot * slot_stride + conv_off;     // [taps-1, C]
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    float acc = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int n = i - (taps - 1) + j;
      const float x = n >= 0 ? to_f(proj[(long long)(first + n) * stride + c]) : cstate[(long long)(taps - 1 + n) * C + c];
      acc = fmaf(conv_w[(long long)c * taps + j], x, acc);
    }
    vals[c] = silu_f(acc);
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float qscale = 1.0f / sqrtf((float)D);
  for (int h = warp; h < 2 * G; h += 4) {        // q heads, then k heads
    const float* v = vals + (long long)h * D;
    float ss = 0.f;
    for (int e = lane; e < D; e += 32) ss = fmaf(v[e], v[e], ss);
    const float inv = 1.0f / sqrtf(warp_sum(ss) + 1e-6f);
    const float mul = h < G ? inv * qscale : inv;
    for (int e = lane; e < D; e += 32) oq[(long long)h * D + e] = v[e] * mul;
  }
  for (int c = 2 * G * D + threadIdx.x; c < C; c += blockDim.x) oq[c] = vals[c];
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float b = ab[(long long)t * ab_stride + h];
    const float a = ab[(long long)t * ab_stride + H + h] + dt_bias[h];
    const float sp = a > 20.f ? a : log1pf(expf(a));
    og[h] = expf(-expf(a_log[h]) * sp);
    og[H + h] = 1.0f / (1.0f + expf(-b));
  }
}

// grid (ceil(Dv / COLS), H, R), 128 threads: COLS = 128 / L columns of S, L adjacent lanes each; lane `sub` of a
// column holds rows d = sub * NPL + i, i < NPL (D <= L NPL).  qkv [T, C] and gb [T, 2H] as delta_prepare left them;
// out [T, H*Dv].  The walk over a request's tokens is one chain of dependent steps per column (decay, dot with k over
// the lanes, write, dot with q), so what matters is the length of a step: a token's operands (k and q of the head's
// group, the block's values, decay and beta) come through shared memory in runs of TB tokens, the next run copied
// (cp.async) while the current one is walked, and the dots run in four interleaved sums.
template <int NPL, int L, int TB>
__global__ void __launch_bounds__(128)
delta_rule_kernel(const float* qkv, const float* gb, const int* row_start, const int* row_slot, float* state,
                  long long slot_stride, float* out, int H, int G, int D, int Dv, int max_slots) {
  constexpr int COLS = 128 / L, DP = NPL * L;
  constexpr int ROWF = (2 * DP + COLS + 2 + 3) / 4 * 4;       // floats of one token in a run: k | q | values | decay, beta
  extern __shared__ __align__(16) float runs[];                // two runs of TB tokens
  const int r = blockIdx.z, h = blockIdx.y;
  const int c0 = blockIdx.x * COLS;
  const int col = c0 + (threadIdx.x / L), sub = threadIdx.x % L;
  if (D < DP)                                    // rows d >= D of k and q are zero and stay so
    for (int i = threadIdx.x; i < 2 * TB * 2 * (DP - D); i += 128) {
      const int s = i / (2 * (DP - D)), e = i - s * 2 * (DP - D);
      runs[s * ROWF + (e < DP - D ? D + e : DP + D + e - (DP - D))] = 0.f;
    }
  pdl_wait();
  pdl_trigger();
  const int slot = row_slot[r];
  if (slot < 0 || slot >= max_slots) return;
  const int first = row_start[r], n = row_start[r + 1] - first;
  const int C = 2 * G * D + H * Dv;
  const int g = h / (H / G);
  const bool live = col < Dv;
  const int colc = live ? col : Dv - 1;          // lanes beyond the last column follow it and write nothing
  float* sp = state + (long long)slot * slot_stride + ((long long)h * Dv + colc) * D;
  float S[NPL], k[NPL], q[NPL];
  // a lane's share of a column in 16-byte accesses where the slots allow it
  const bool vec = (D & 3) == 0 && (slot_stride & 3) == 0 && (((uintptr_t)state) & 15) == 0;
  if (vec) {
#pragma unroll
    for (int i = 0; i < NPL; i += 4) {
      const int d = sub * NPL + i;
      const float4 x = d < D ? *reinterpret_cast<const float4*>(sp + d) : make_float4(0.f, 0.f, 0.f, 0.f);
      S[i] = x.x; S[i + 1] = x.y; S[i + 2] = x.z; S[i + 3] = x.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int d = sub * NPL + i;
      S[i] = d < D ? sp[d] : 0.f;
    }
  }
  const long long qoff = (long long)g * D, koff = (long long)(G + g) * D, voff = (long long)2 * G * D + (long long)h * Dv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // 16-byte copies where a token's k and q start on 16 bytes in global memory, else 4-byte ones
  const bool wide = (D & 3) == 0 && (C & 3) == 0 && (((uintptr_t)qkv) & 15) == 0;
  auto cp = [](float* dst, const float* src, int bytes) {
    const unsigned sa = (unsigned)__cvta_generic_to_shared(dst);
    if (bytes == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(src));
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(sa), "l"(src));
  };
  auto copy_run = [&](int run) {                 // tokens [run * TB, ...) of the request into buffer run & 1: a warp per token
    float* dst0 = runs + (run & 1) * TB * ROWF;
    const int t0 = run * TB, cnt = min(TB, n - t0);
    for (int s = warp; s < cnt; s += 4) {
      const float* row = qkv + (long long)(first + t0 + s) * C;
      float* dst = dst0 + s * ROWF;
      if (wide) {
        for (int d = 4 * lane; d < D; d += 128) {
          cp(dst + d, row + koff + d, 16);
          cp(dst + DP + d, row + qoff + d, 16);
        }
      } else {
        for (int d = lane; d < D; d += 32) {
          cp(dst + d, row + koff + d, 4);
          cp(dst + DP + d, row + qoff + d, 4);
        }
      }
      for (int e = lane; e < COLS; e += 32) cp(dst + 2 * DP + e, row + voff + min(c0 + e, Dv - 1), 4);
      if (lane < 2) cp(dst + 2 * DP + COLS + lane, gb + (long long)(first + t0 + s) * 2 * H + lane * H + h, 4);   // decay, beta
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  const int n_runs = (n + TB - 1) / TB;
  __syncthreads();                               // the zeros are written before any copy lands
  if (n_runs > 0) copy_run(0);
  for (int run = 0; run < n_runs; ++run) {
    if (run + 1 < n_runs) {
      copy_run(run + 1);
      asm volatile("cp.async.wait_group 1;\n" ::);
    } else {
      asm volatile("cp.async.wait_group 0;\n" ::);
    }
    __syncthreads();
    const float* buf = runs + (run & 1) * TB * ROWF;
    const int cnt = min(TB, n - run * TB);
#pragma unroll 2
    for (int s = 0; s < cnt; ++s) {
      const float* tokp = buf + s * ROWF;
#pragma unroll
      for (int i = 0; i < NPL; i += 4) {           // 16-byte loads: a run's rows and a lane's share start on 16 bytes
        const float4 k4 = *reinterpret_cast<const float4*>(tokp + sub * NPL + i);
        const float4 q4 = *reinterpret_cast<const float4*>(tokp + DP + sub * NPL + i);
        k[i] = k4.x; k[i + 1] = k4.y; k[i + 2] = k4.z; k[i + 3] = k4.w;
        q[i] = q4.x; q[i + 1] = q4.y; q[i + 2] = q4.z; q[i + 3] = q4.w;
      }
      const float v = tokp[2 * DP + (threadIdx.x / L)], gd = tokp[2 * DP + COLS], beta = tokp[2 * DP + COLS + 1];
      float dp[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        S[i] *= gd;
        dp[i & 3] = fmaf(S[i], k[i], dp[i & 3]);
      }
      float dot = (dp[0] + dp[1]) + (dp[2] + dp[3]);
#pragma unroll
      for (int o = 1; o < L; o <<= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
      const float u = beta * (v - dot);
      float op[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        S[i] = fmaf(k[i], u, S[i]);
        op[i & 3] = fmaf(S[i], q[i], op[i & 3]);
      }
      float o = (op[0] + op[1]) + (op[2] + op[3]);
#pragma unroll
      for (int x = 1; x < L; x <<= 1) o += __shfl_xor_sync(0xffffffffu, o, x);
      if (live && sub == 0) out[(long long)(first + run * TB + s) * H * Dv + (long long)h * Dv + col] = o;
    }
    __syncthreads();                             // the run is walked: its buffer may take the run after the next
  }
  if (live && vec) {
#pragma unroll
    for (int i = 0; i < NPL; i += 4) {
      const int d = sub * NPL + i;
      if (d < D) *reinterpret_cast<float4*>(sp + d) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
    }
  } else if (live) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int d = sub * NPL + i;
      if (d < D) sp[d] = S[i];
    }
  }
}

// One warp per (token, head): out[t, h, :] = o / sqrt(mean(o^2) + eps) * w * silu(gate[t, h, :]).
template <typename T>
__global__ void __launch_bounds__(128)
gated_rmsnorm_kernel(const float* o, const T* gate, long long gate_stride, const float* __restrict__ w, T* out,
                     long long out_stride, long long n_items, int H, int Dv, float eps) {
  pdl_wait();
  pdl_trigger();
  const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= n_items) return;
  const long long t = item / H;
  const int h = (int)(item - t * H);
  const float* op = o + (t * H + h) * Dv;
  const T* gp = gate + t * gate_stride + (long long)h * Dv;
  T* dst = out + t * out_stride + (long long)h * Dv;
  float ss = 0.f;
  for (int e = lane; e < Dv; e += 32) ss = fmaf(op[e], op[e], ss);
  const float rstd = 1.0f / sqrtf(warp_sum(ss) / (float)Dv + eps);
  for (int e = lane; e < Dv; e += 32) dst[e] = from_f<T>(op[e] * rstd * w[e] * silu_f(to_f(gp[e])));
}
}  // namespace

FMX_EXPORT int fmx_delta_prepare(const void* proj, long long stride, const float* ab, long long ab_stride,
                                 const float* conv_w, const float* a_log, const float* dt_bias, const int* token_row,
                                 const int* row_start, const int* row_slot, float* state, long long slot_stride,
                                 long long conv_off, float* out_qkv, float* out_gb, int T, int R, int H, int G, int D, int Dv,
                                 int taps, int max_slots, int dtype, int* status, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || R <= 0 || H <= 0 || G <= 0 || H % G || D <= 0 || Dv <= 0 || taps < 1 || taps > MAX_TAPS)
    return fmx_fail("fmx_delta_prepare: bad sizes T=%d R=%d H=%d G=%d D=%d Dv=%d taps=%d", T, R, H, G, D, Dv, taps);
  const int C = 2 * G * D + H * Dv;
  if (stride < C || ab_stride < 2 * H) return fmx_fail("fmx_delta_prepare: rows too narrow");
  const size_t smem = (size_t)C * sizeof(float);
  if (smem > 200 * 1024) return fmx_fail("fmx_delta_prepare: %d channels do not fit shared memory", C);
#define FMX_DELTA_PREP(TT)                                                                                             \
  do {                                                                                                                 \
    if (smem > 48 * 1024)                                                                                              \
      cudaFuncSetAttribute(delta_prepare_kernel<TT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);         \
    fmx_launch(delta_prepare_kernel<TT>, dim3(T), dim3(128), smem, stream, (const TT*)proj, stride, ab, ab_stride, conv_w, \
               a_log, dt_bias, token_row, row_start, row_slot, (const float*)state, slot_stride, conv_off, out_qkv,    \
               out_gb, H, G, D, Dv, taps, R, max_slots, status);                                                       \
    fmx_launch(conv_state_update_kernel<TT>, dim3((C + 127) / 128, R), dim3(128), 0, stream, (const TT*)proj, stride,  \
               row_start, row_slot, state, slot_stride, conv_off, C, taps, max_slots);                                 \
  } while (0)
  if (dtype == FMX_F32)
    FMX_DELTA_PREP(float);
  else if (dtype == FMX_BF16)
    FMX_DELTA_PREP(bf16);
  else
    return fmx_fail("fmx_delta_prepare: unknown dtype %d", dtype);
#undef FMX_DELTA_PREP
  FMX_LAUNCH_CHECK();
  return 0;
}

FMX_EXPORT int fmx_delta_rule(const float* qkv, const float* gb, const int* row_start, const int* row_slot, float* state,
                              long long slot_stride, float* out, int R, int H, int G, int D, int Dv, int max_slots,
                              int lanes, cudaStream_t stream) {
  if (R == 0) return 0;
  if (R < 0 || H <= 0 || G <= 0 || H % G || D <= 0 || Dv <= 0 || D > 256)
    return fmx_fail("fmx_delta_rule: bad sizes R=%d H=%d G=%d D=%d Dv=%d", R, H, G, D, Dv);
  if (H > 65535 || R > 65535) return fmx_fail("fmx_delta_rule: batch too large");
#define FMX_DELTA_RULE(NPL, L, TB)                                                                                     \
  do {                                                                                                                 \
    constexpr int cols = 128 / (L), rowf = (2 * (NPL) * (L) + cols + 2 + 3) / 4 * 4;                                   \
    const dim3 grid((Dv + cols - 1) / cols, H, R);                                                                     \
    constexpr size_t smem = (size_t)2 * (TB) * rowf * sizeof(float);                                                   \
    if (smem > 48 * 1024)                                                                                              \
      cudaFuncSetAttribute(delta_rule_kernel<NPL, L, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
    fmx_launch(delta_rule_kernel<NPL, L, TB>, grid, dim3(128), smem, stream, qkv, gb, row_start, row_slot, state,      \
               slot_stride, out, H, G, D, Dv, max_slots);                                                              \
  } while (0)
  // Lanes per column: few lanes make a step's sums over lanes short, many lanes make its dots short and give the
  // grid more warps.  `lanes` = 0 leaves the choice here.
  // Measured (us for 2,048 tokens of one request, 32 heads): dim 64: 8 lanes 524, 16 lanes 549, 4 lanes 600; dim 128: 8 lanes
  // 1,345, 16 lanes 963: eight rows of state per lane.
  if (lanes == 0) lanes = D <= 64 ? 8 : D <= 128 ? 16 : 32;
  if (lanes != 2 && lanes != 4 && lanes != 8 && lanes != 16 && lanes != 32)
    return fmx_fail("fmx_delta_rule: 2, 4, 8, 16 or 32 lanes per column, not %d", lanes);
  const int per_lane = (D + lanes - 1) / lanes;
  if (per_lane > 32) return fmx_fail("fmx_delta_rule: %d rows of state are too many for %d lanes per column", D, lanes);
#define FMX_DELTA_LANES(L)                      \
  do {                                          \
    if (per_lane <= 4) FMX_DELTA_RULE(4, L, 16);       \
    else if (per_lane <= 8) FMX_DELTA_RULE(8, L, 16);  \
    else if (per_lane <= 16) FMX_DELTA_RULE(16, L, 16); \
    else FMX_DELTA_RULE(32, L, 8);              \
  } while (0)
  if (lanes == 2) FMX_DELTA_LANES(2);
  else if (lanes == 4) FMX_DELTA_LANES(4);
  else if (lanes == 8) FMX_DELTA_LANES(8);
  else if (lanes == 16) FMX_DELTA_LANES(16);
  else FMX_DELTA_LANES(32);
#undef FMX_DELTA_LANES
#undef FMX_DELTA_RULE
  FMX_LAUNCH_CHECK();
  return 0;
}

FMX_EXPORT int fmx_gated_rmsnorm(const float* o, const void* gate, long long gate_stride, const float* w, void* out,
                                 long long out_stride, int T, int H, int Dv, float eps, int dtype, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || H <= 0 || Dv <= 0) return fmx_fail("fmx_gated_rmsnorm: bad sizes T=%d H=%d Dv=%d", T, H, Dv);
  const long long items = (long long)T * H;
  const long long grid = (items + 3) / 4;
  if (grid > 2147483647LL) return fmx_fail("fmx_gated_rmsnorm: batch too large");
  if (dtype == FMX_F32)
    fmx_launch(gated_rmsnorm_kernel<float>, dim3((unsigned)grid), dim3(128), 0, stream, o, (const float*)gate, gate_stride, w,
               (float*)out, out_stride, items, H, Dv, eps);
  else if (dtype == FMX_BF16)
    fmx_launch(gated_rmsnorm_kernel<bf16>, dim3((unsigned)grid), dim3(128), 0, stream, o, (const bf16*)gate, gate_stride, w,
               (bf16*)out, out_stride, items, H, Dv, eps);
  else
    return fmx_fail("fmx_gated_rmsnorm: unknown dtype %d", dtype);
  FMX_LAUNCH_CHECK();
  return 0;
}
