// A state-space recurrence with a matrix of state per head and a scalar decay per head and token.
//
// Per head h, with x (size P), B and C (size N, of the head's group), a step size dt > 0 and a decay a in (0, 1),
// a token does
//     S <- a S + dt B x^T;   y = S^T C + D_h x,
// S [N, P] in 32-bit in a state slot of the request, carried from step to step; so are the last taps-1 inputs of
// the short causal convolution that x, B and C pass through.
//
// Three kernels (and conv_state_update of conv_state.cuh):
//   ssm_prepare          per token: convolution with bias + SiLU of the projected x | B | C channels (inputs before the
//                        portion's start come from the slot's convolution state), dt = softplus(dt + dt_bias) without
//                        a clamp, a = exp(-exp(A_log) dt).
//   ssm_scan             the recurrence.  Columns of S are independent (column j needs x_j only), so a column is given
//                        to 8 to 32 adjacent lanes that hold some of its N values each in registers; a request's tokens
//                        are walked in order, their operands staged through shared memory a run of tokens ahead.  The
//                        chain from token to token is one multiply-add per value of state; the read-out's sum over the
//                        lanes hangs off it.
//   gated_group_rmsnorm  y * SiLU(z), then divided by its root mean square in equal parts of the row, times a weight.
//
// A slot's state is one run of 32-bit floats: S^T of every head, [H, P, N], and then the convolution inputs,
// [taps-1, C], C = H*P + 2*G*N.  Everything is 32-bit but the projection that comes in and the activations that go
// out.  No sum's order depends on how a request's tokens were cut into steps or on what else is in the batch.
#include <math.h>
#include "common.cuh"
#include "conv_state.cuh"

namespace {
constexpr int PREP_CHANNELS = 512;               // channels of a token that one block of ssm_prepare takes
// proj [T, stride]: z (H*P) | x (H*P) | B (G*N) | C (G*N) | dt (H).  out_xbc [T, C] 32-bit; out_dd [T, 2H]: dt | decay.
template <typename T>
__global__ void __launch_bounds__(128)
ssm_prepare_kernel(const T* __restrict__ proj, long long stride, const float* __restrict__ conv_w,
                   const float* __restrict__ conv_b, const float* __restrict__ a_log, const float* __restrict__ dt_bias,
                   const int* __restrict__ token_row, const int* __restrict__ row_start, const int* __restrict__ row_slot,
                   const float* __restrict__ state, long long slot_stride, long long conv_off, float* __restrict__ out_xbc,
                   float* __restrict__ out_dd, int H, int C, int inner, int taps, int R, int max_slots, int* status) {
  pdl_wait();
  pdl_trigger();
  // grid (T, ceil(C / PREP_CHANNELS)): a block takes a run of a token's channels, so that a step of few tokens still
  // fills the GPU; the blocks of the first run also take the token's step sizes and decays
  const int t = blockIdx.x;
  const int c_lo = blockIdx.y * PREP_CHANNELS, c_hi = min(C, c_lo + PREP_CHANNELS);
  const int r = token_row[t];
  float* ox = out_xbc + (long long)t * C;
  float* od = out_dd + (long long)t * 2 * H;
  const int slot = (r >= 0 && r < R) ? row_slot[r] : -1;
  if (slot < 0 || slot >= max_slots) {          // a padding row of a captured step, or a bad row: nothing to do
    if (blockIdx.y == 0) {
      if (r < 0 || r >= R) { if (threadIdx.x == 0) fmx_set_status(status, FMX_BAD_ROW, r, t); }
      else if (slot >= max_slots && threadIdx.x == 0) fmx_set_status(status, FMX_BAD_SLOT, slot, t);
      for (int c = threadIdx.x; c < 2 * H; c += blockDim.x) od[c] = 0.f;
    }
    for (int c = c_lo + threadIdx.x; c < c_hi; c += blockDim.x) ox[c] = 0.f;
    return;
  }
  const int first = row_start[r];
  const int i = t - first;                       // the token's place in its portion
  const float* cstate = state + (long long)slot * slot_stride + conv_off;     // [taps-1, C]
  const T* in = proj + inner;                    // the convolution's channels start behind z
#pragma unroll 4
  for (int c = c_lo + threadIdx.x; c < c_hi; c += blockDim.x) {
    float acc = conv_b[c];
    for (int j = 0; j < taps; ++j) {
      const int n = i - (taps - 1) + j;
      const float x = n >= 0 ? to_f(in[(long long)(first + n) * stride + c]) : cstate[(long long)(taps - 1 + n) * C + c];
      acc = fmaf(conv_w[(long long)c * taps + j], x, acc);
    }
    ox[c] = silu_f(acc);
  }
  if (blockIdx.y != 0) return;
  for (int h = threadIdx.x; h < H; h += blockDim.x) {
    const float a = to_f(proj[(long long)t * stride + inner + C + h]) + dt_bias[h];
    const float dt = a > 20.f ? a : log1pf(expf(a));
    od[h] = dt;
    od[H + h] = expf(-expf(a_log[h]) * dt);
  }
}

// grid (ceil(P / COLS), H, R), 128 threads: COLS = 128 / L columns of S, L adjacent lanes each; lane `sub` of a column
// holds rows n = sub * NPL + i, i < NPL (N <= L NPL).  xbc [T, C] and dd [T, 2H] as ssm_prepare left them; out [T, H*P].
// A token's operands (B and C of the head's group, the block's x values, dt and decay) come through shared memory in
// runs of TB tokens, the next run copied (cp.async) while the current one is walked.
template <int NPL, int L, int TB>
__global__ void __launch_bounds__(128)
ssm_scan_kernel(const float* xbc, const float* dd, const float* __restrict__ d_skip, const int* row_start,
                const int* row_slot, float* state, long long slot_stride, float* out, int H, int G, int N, int P,
                int max_slots) {
  constexpr int COLS = 128 / L, NP = NPL * L;
  constexpr int ROWF = (2 * NP + COLS + 2 + 3) / 4 * 4;       // floats of one token in a run: B | C | x values | dt, decay
  extern __shared__ __align__(16) float runs[];                // two runs of TB tokens
  const int r = blockIdx.z, h = blockIdx.y;
  const int c0 = blockIdx.x * COLS;
  const int col = c0 + (threadIdx.x / L), sub = threadIdx.x % L;
  if (N < NP)                                    // rows n >= N of B and C are zero and stay so
    for (int i = threadIdx.x; i < 2 * TB * 2 * (NP - N); i += 128) {
      const int s = i / (2 * (NP - N)), e = i - s * 2 * (NP - N);
      runs[s * ROWF + (e < NP - N ? N + e : NP + N + e - (NP - N))] = 0.f;
    }
  pdl_wait();
  pdl_trigger();
  const int slot = row_slot[r];
  if (slot < 0 || slot >= max_slots) return;
  const int first = row_start[r], n = row_start[r + 1] - first;
  const int inner = H * P, C = inner + 2 * G * N;
  const int g = h / (H / G);
  const bool live = col < P;
  const int colc = live ? col : P - 1;           // lanes beyond the last column follow it and write nothing
  float* sp = state + (long long)slot * slot_stride + ((long long)h * P + colc) * N;
  float S[NPL];
  const bool vec = (N & 3) == 0 && (slot_stride & 3) == 0 && (((uintptr_t)state) & 15) == 0;
  if (vec) {
#pragma unroll
    for (int i = 0; i < NPL; i += 4) {
      const int d = sub * NPL + i;
      const float4 x = d < N ? *reinterpret_cast<const float4*>(sp + d) : make_float4(0.f, 0.f, 0.f, 0.f);
      S[i] = x.x; S[i + 1] = x.y; S[i + 2] = x.z; S[i + 3] = x.w;
    }
  } else {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int d = sub * NPL + i;
      S[i] = d < N ? sp[d] : 0.f;
    }
  }
  const long long xoff = (long long)h * P, boff = (long long)inner + (long long)g * N,
                  coff = (long long)inner + (long long)(G + g) * N;
  const float skip = d_skip[h];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // 16-byte copies where a token's B and C start on 16 bytes in global memory, else 4-byte ones
  const bool wide = (N & 3) == 0 && (C & 3) == 0 && (inner & 3) == 0 && (((uintptr_t)xbc) & 15) == 0;
  auto cp = [](float* dst, const float* src, int bytes) {
    const unsigned sa = (unsigned)__cvta_generic_to_shared(dst);
    if (bytes == 16) asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(sa), "l"(src));
    else asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(sa), "l"(src));
  };
  auto copy_run = [&](int run) {                 // tokens [run * TB, ...) of the request into buffer run & 1: a warp per token
    float* dst0 = runs + (run & 1) * TB * ROWF;
    const int t0 = run * TB, cnt = min(TB, n - t0);
    for (int s = warp; s < cnt; s += 4) {
      const float* row = xbc + (long long)(first + t0 + s) * C;
      float* dst = dst0 + s * ROWF;
      if (wide) {
        for (int d = 4 * lane; d < N; d += 128) {
          cp(dst + d, row + boff + d, 16);
          cp(dst + NP + d, row + coff + d, 16);
        }
      } else {
        for (int d = lane; d < N; d += 32) {
          cp(dst + d, row + boff + d, 4);
          cp(dst + NP + d, row + coff + d, 4);
        }
      }
      for (int e = lane; e < COLS; e += 32) cp(dst + 2 * NP + e, row + xoff + min(c0 + e, P - 1), 4);
      if (lane < 2) cp(dst + 2 * NP + COLS + lane, dd + (long long)(first + t0 + s) * 2 * H + lane * H + h, 4);   // dt, decay
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
    // a token's operands out of the run's buffer: this lane's rows of B and C, the column's x, the head's dt and decay
    struct Operands { float b[NPL], c[NPL], x, dt, decay; };
    auto fetch = [&](int s, Operands& t) {
      const float* tokp = buf + s * ROWF;
#pragma unroll
      for (int i = 0; i < NPL; i += 4) {           // 16-byte loads: a run's rows and a lane's share start on 16 bytes
        const float4 b4 = *reinterpret_cast<const float4*>(tokp + sub * NPL + i);
        const float4 c4 = *reinterpret_cast<const float4*>(tokp + NP + sub * NPL + i);
        t.b[i] = b4.x; t.b[i + 1] = b4.y; t.b[i + 2] = b4.z; t.b[i + 3] = b4.w;
        t.c[i] = c4.x; t.c[i + 1] = c4.y; t.c[i + 2] = c4.z; t.c[i + 3] = c4.w;
      }
      t.x = tokp[2 * NP + (threadIdx.x / L)];
      t.dt = tokp[2 * NP + COLS];
      t.decay = tokp[2 * NP + COLS + 1];
    };
    // one token: this lane's rows of the column move on, and it returns its part of the read-out S^T C
    auto advance = [&](const Operands& t) -> float {
      const float u = t.dt * t.x;
      float op[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int i = 0; i < NPL; ++i) {
        S[i] = fmaf(t.b[i], u, S[i] * t.decay);
        op[i & 3] = fmaf(S[i], t.c[i], op[i & 3]);
      }
      return (op[0] + op[1]) + (op[2] + op[3]);
    };
    if (L <= TB && n > 1) {
     if constexpr (L <= TB) {
      // L tokens at a time: the lanes' parts of L read-outs are added up across the column's L lanes together, each
      // round halving what a lane holds (L - 1 exchanges for L tokens, none waiting for another), and lane j is left
      // with token j's sum, which it writes.  The pairs of lanes that meet in a round are the same for every token,
      // so a token's sum does not depend on its place in the run.
      for (int gb = 0; gb < cnt; gb += L) {
        float v[L];
        Operands cur, nxt;                         // the next token's operands are on their way while this one is walked
        fetch(gb, cur);
#pragma unroll
        for (int j = 0; j < L; ++j) {
          if (j + 1 < L && gb + j + 1 < cnt) fetch(gb + j + 1, nxt);
          v[j] = gb + j < cnt ? advance(cur) : 0.f;
          if (j + 1 < L) cur = nxt;
        }
#pragma unroll
        for (int d = L / 2; d >= 1; d >>= 1) {
          const bool upper = (sub & d) != 0;
#pragma unroll
          for (int j = 0; j < d; ++j) {
            const float give = upper ? v[j] : v[j + d], keep = upper ? v[j + d] : v[j];
            v[j] = keep + __shfl_xor_sync(0xffffffffu, give, d);
          }
        }
        const int s = gb + sub;
        if (live && s < cnt) {
          const float x = buf[s * ROWF + 2 * NP + (threadIdx.x / L)];
          out[(long long)(first + run * TB + s) * inner + (long long)h * P + col] = fmaf(skip, x, v[0]);
        }
      }
     }
    } else {
      // a row of one token (and columns of 32 lanes): every lane gets the sum, by the same pairs in the same order
#pragma unroll 2
      for (int s = 0; s < cnt; ++s) {
        Operands cur;
        fetch(s, cur);
        float o = advance(cur);
#pragma unroll
        for (int k = L / 2; k >= 1; k >>= 1) o += __shfl_xor_sync(0xffffffffu, o, k);
        const float x = buf[s * ROWF + 2 * NP + (threadIdx.x / L)];
        if (live && sub == 0) out[(long long)(first + run * TB + s) * inner + (long long)h * P + col] = fmaf(skip, x, o);
      }
    }
    __syncthreads();                             // the run is walked: its buffer may take the run after the next
  }
  if (live && vec) {
#pragma unroll
    for (int i = 0; i < NPL; i += 4) {
      const int d = sub * NPL + i;
      if (d < N) *reinterpret_cast<float4*>(sp + d) = make_float4(S[i], S[i + 1], S[i + 2], S[i + 3]);
    }
  } else if (live) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int d = sub * NPL + i;
      if (d < N) sp[d] = S[i];
    }
  }
}

// One block per (token, part): v = y * silu(z) over the part's n values, out = v / sqrt(mean(v^2) + eps) * w.
template <typename T>
__global__ void __launch_bounds__(128)
gated_group_rmsnorm_kernel(const float* y, const T* z, long long z_stride, const float* __restrict__ w, T* out,
                           long long out_stride, int groups, int n, float eps) {
  pdl_wait();
  pdl_trigger();
  const long long t = blockIdx.x / groups;
  const int gi = blockIdx.x - (int)(t * groups);
  const float* yp = y + (t * groups + gi) * n;
  const T* zp = z + t * z_stride + (long long)gi * n;
  T* dst = out + t * out_stride + (long long)gi * n;
  const float* wp = w + (long long)gi * n;
  float ss = 0.f;
  for (int e = threadIdx.x; e < n; e += blockDim.x) {
    const float v = yp[e] * silu_f(to_f(zp[e]));
    ss = fmaf(v, v, ss);
  }
  const float rstd = 1.0f / sqrtf(block_sum<128>(ss) / (float)n + eps);
  for (int e = threadIdx.x; e < n; e += blockDim.x) dst[e] = from_f<T>(yp[e] * silu_f(to_f(zp[e])) * rstd * wp[e]);
}
}  // namespace

FMX_EXPORT int fmx_ssm_prepare(const void* proj, long long stride, const float* conv_w, const float* conv_b,
                               const float* a_log, const float* dt_bias, const int* token_row, const int* row_start,
                               const int* row_slot, float* state, long long slot_stride, long long conv_off, float* out_xbc,
                               float* out_dd, int T, int R, int H, int G, int N, int P, int taps, int max_slots, int dtype,
                               int* status, cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || R <= 0 || H <= 0 || G <= 0 || H % G || N <= 0 || P <= 0 || taps < 1 || taps > MAX_TAPS)
    return fmx_fail("fmx_ssm_prepare: bad sizes T=%d R=%d H=%d G=%d N=%d P=%d taps=%d", T, R, H, G, N, P, taps);
  const int inner = H * P, C = inner + 2 * G * N;
  if (stride < 2 * inner + 2 * G * N + H) return fmx_fail("fmx_ssm_prepare: rows too narrow");
#define FMX_SSM_PREP(TT)                                                                                               \
  do {                                                                                                                 \
    fmx_launch(ssm_prepare_kernel<TT>, dim3(T, (C + PREP_CHANNELS - 1) / PREP_CHANNELS), dim3(128), 0, stream, (const TT*)proj, stride, conv_w, conv_b, a_log,  \
               dt_bias, token_row, row_start, row_slot, (const float*)state, slot_stride, conv_off, out_xbc, out_dd, H, C, \
               inner, taps, R, max_slots, status);                                                                     \
    fmx_launch(conv_state_update_kernel<TT>, dim3((C + 127) / 128, R), dim3(128), 0, stream, (const TT*)proj + inner,  \
               stride, row_start, row_slot, state, slot_stride, conv_off, C, taps, max_slots);                         \
  } while (0)
  if (dtype == FMX_F32)
    FMX_SSM_PREP(float);
  else if (dtype == FMX_BF16)
    FMX_SSM_PREP(bf16);
  else
    return fmx_fail("fmx_ssm_prepare: unknown dtype %d", dtype);
#undef FMX_SSM_PREP
  FMX_LAUNCH_CHECK();
  return 0;
}

FMX_EXPORT int fmx_ssm_scan(const float* xbc, const float* dd, const float* d_skip, const int* row_start,
                            const int* row_slot, float* state, long long slot_stride, float* out, int R, int H, int G, int N,
                            int P, int max_slots, int lanes, cudaStream_t stream) {
  if (R == 0) return 0;
  if (R < 0 || H <= 0 || G <= 0 || H % G || N <= 0 || P <= 0 || N > 1024)
    return fmx_fail("fmx_ssm_scan: bad sizes R=%d H=%d G=%d N=%d P=%d", R, H, G, N, P);
  if (H > 65535 || R > 65535) return fmx_fail("fmx_ssm_scan: batch too large");
#define FMX_SSM_SCAN(NPL, L, TB)                                                                                       \
  do {                                                                                                                 \
    constexpr int cols = 128 / (L), rowf = (2 * (NPL) * (L) + cols + 2 + 3) / 4 * 4;                                   \
    const dim3 grid((P + cols - 1) / cols, H, R);                                                                      \
    constexpr size_t smem = (size_t)2 * (TB) * rowf * sizeof(float);                                                   \
    if (smem > 48 * 1024)                                                                                              \
      cudaFuncSetAttribute(ssm_scan_kernel<NPL, L, TB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
    fmx_launch(ssm_scan_kernel<NPL, L, TB>, grid, dim3(128), smem, stream, xbc, dd, d_skip, row_start, row_slot, state, \
               slot_stride, out, H, G, N, P, max_slots);                                                               \
  } while (0)
  // lanes per column: eight values of state per lane where the state's size allows
  if (lanes == 0) lanes = N <= 64 ? 8 : N <= 128 ? 16 : 32;
  if (lanes != 2 && lanes != 4 && lanes != 8 && lanes != 16 && lanes != 32)
    return fmx_fail("fmx_ssm_scan: 2, 4, 8, 16 or 32 lanes per column, not %d", lanes);
  const int per_lane = (N + lanes - 1) / lanes;
  if (per_lane > 32) return fmx_fail("fmx_ssm_scan: %d rows of state are too many for %d lanes per column", N, lanes);
#define FMX_SSM_LANES(L)                        \
  do {                                          \
    if (per_lane <= 4) FMX_SSM_SCAN(4, L, 16);         \
    else if (per_lane <= 8) FMX_SSM_SCAN(8, L, 16);    \
    else if (per_lane <= 16) FMX_SSM_SCAN(16, L, 16);  \
    else FMX_SSM_SCAN(32, L, 8);                \
  } while (0)
  if (lanes == 2) FMX_SSM_LANES(2);
  else if (lanes == 4) FMX_SSM_LANES(4);
  else if (lanes == 8) FMX_SSM_LANES(8);
  else if (lanes == 16) FMX_SSM_LANES(16);
  else FMX_SSM_LANES(32);
#undef FMX_SSM_LANES
#undef FMX_SSM_SCAN
  FMX_LAUNCH_CHECK();
  return 0;
}

// y [T, groups * n] 32-bit, z and out of `dtype` in rows that may be slices of wider buffers, w [groups * n].
FMX_EXPORT int fmx_gated_group_rmsnorm(const float* y, const void* z, long long z_stride, const float* w, void* out,
                                       long long out_stride, int T, int groups, int n, float eps, int dtype,
                                       cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || groups <= 0 || n <= 0) return fmx_fail("fmx_gated_group_rmsnorm: bad sizes T=%d groups=%d n=%d", T, groups, n);
  const long long grid = (long long)T * groups;
  if (grid > 2147483647LL) return fmx_fail("fmx_gated_group_rmsnorm: batch too large");
  if (dtype == FMX_F32)
    fmx_launch(gated_group_rmsnorm_kernel<float>, dim3((unsigned)grid), dim3(128), 0, stream, y, (const float*)z, z_stride, w,
               (float*)out, out_stride, groups, n, eps);
  else if (dtype == FMX_BF16)
    fmx_launch(gated_group_rmsnorm_kernel<bf16>, dim3((unsigned)grid), dim3(128), 0, stream, y, (const bf16*)z, z_stride, w,
               (bf16*)out, out_stride, groups, n, eps);
  else
    return fmx_fail("fmx_gated_group_rmsnorm: unknown dtype %d", dtype);
  FMX_LAUNCH_CHECK();
  return 0;
}
