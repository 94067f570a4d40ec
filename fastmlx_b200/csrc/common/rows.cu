// Two small row-wise kernels that mixers with a latent or a gate need.
//
// rmsnorm_rows: a slice of every row divided by its root mean square and multiplied by a weight, x / sqrt(mean(x^2)
// + eps) * w, in 32-bit, written either to the same row of a dense output or to the row that a map names (the
// cache slot of the token: how a normalised latent goes straight into its page).  The sum of squares is taken in an
// order that depends on the slice's width alone.
//
// sigmoid_gate: o[t, j] *= sigmoid(g[t, j / group]) in 32-bit: group = 1 gates element by element, group = the
// head's width gates a head by one value.
//
// rmsnorm_pair_mean: out = (a / rms(a) * wa + b / rms(b) * wb) / 2, each row of a and of b divided by its own root mean
// square: how a layer joins two mixers that ran side by side on the same input.
#include <math.h>
#include "common.cuh"

namespace {
constexpr int NORM_BLOCK = 128;

template <typename TI, typename TO>
__global__ void __launch_bounds__(NORM_BLOCK)
rmsnorm_pair_mean_kernel(const TI* a, long long a_stride, const TI* b, long long b_stride, const float* __restrict__ wa,
                         const float* __restrict__ wb, float eps, TO* out, long long out_stride, int n) {
  pdl_wait();
  pdl_trigger();
  const long long t = blockIdx.x;
  const TI* pa = a + t * a_stride;
  const TI* pb = b + t * b_stride;
  float sa = 0.f, sb = 0.f;
  for (int e = threadIdx.x; e < n; e += NORM_BLOCK) {
    const float x = to_f(pa[e]), y = to_f(pb[e]);
    sa = fmaf(x, x, sa);
    sb = fmaf(y, y, sb);
  }
  const float ma = 1.0f / sqrtf(block_sum<NORM_BLOCK>(sa) / (float)n + eps);
  const float mb = 1.0f / sqrtf(block_sum<NORM_BLOCK>(sb) / (float)n + eps);
  TO* dst = out + t * out_stride;
  for (int e = threadIdx.x; e < n; e += NORM_BLOCK)
    dst[e] = from_f<TO>(0.5f * (to_f(pa[e]) * ma * wa[e] + to_f(pb[e]) * mb * wb[e]));
}

template <typename TI, typename TO>
__global__ void __launch_bounds__(NORM_BLOCK)
rmsnorm_rows_kernel(const TI* x, long long x_stride, const float* __restrict__ w, float eps, TO* out, long long out_stride,
                    const long long* row_map, long long max_rows, int n, int* status) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  const TI* src = x + (long long)t * x_stride;
  float ss = 0.f;
  for (int e = threadIdx.x; e < n; e += NORM_BLOCK) {
    const float v = to_f(src[e]);
    ss = fmaf(v, v, ss);
  }
  const float mul = 1.0f / sqrtf(block_sum<NORM_BLOCK>(ss) / (float)n + eps);
  long long row = t;
  if (row_map != nullptr) {
    row = row_map[t];
    if (row < 0) return;                         // a token that is stored nowhere (a padding row)
    if (row >= max_rows) {
      if (threadIdx.x == 0) fmx_set_status(status, FMX_BAD_SLOT, row, t);
      return;
    }
  }
  TO* dst = out + row * out_stride;
  for (int e = threadIdx.x; e < n; e += NORM_BLOCK) dst[e] = from_f<TO>(to_f(src[e]) * mul * w[e]);
}

template <typename TO, typename TG>
__global__ void sigmoid_gate_kernel(TO* o, long long o_stride, const TG* g, long long g_stride, long long rows, int cols,
                                    int group) {
  pdl_wait();
  pdl_trigger();
  const long long n = rows * cols;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / cols;
    const int c = (int)(idx - r * cols);
    const float z = to_f(g[r * g_stride + c / group]);
    TO* p = o + r * o_stride + c;
    *p = from_f<TO>(to_f(*p) / (1.0f + expf(-z)));
  }
}
// The same for a bfloat16 output and a 32-bit gate, four columns per thread (one gate value where a group holds them).
__global__ void sigmoid_gate_vec_kernel(bf16* o, long long o_stride, const float* g, long long g_stride, long long rows, int cols,
                                        int group) {
  pdl_wait();
  pdl_trigger();
  const int c4 = cols / 4;
  const long long n = rows * c4;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const long long r = idx / c4;
    const int c = (int)(idx - r * c4) * 4;
    float z[4];
    if (group == 1) {
      const float4 v = *reinterpret_cast<const float4*>(g + r * g_stride + c);
      z[0] = v.x; z[1] = v.y; z[2] = v.z; z[3] = v.w;
    } else {
      z[0] = z[1] = z[2] = z[3] = g[r * g_stride + c / group];
    }
    uint2* p = reinterpret_cast<uint2*>(o + r * o_stride + c);
    uint2 u = *p;
    float2 a = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u.x)), b = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u.y));
    __nv_bfloat162 lo = __floats2bfloat162_rn(a.x / (1.0f + expf(-z[0])), a.y / (1.0f + expf(-z[1])));
    __nv_bfloat162 hi = __floats2bfloat162_rn(b.x / (1.0f + expf(-z[2])), b.y / (1.0f + expf(-z[3])));
    u.x = *reinterpret_cast<unsigned*>(&lo);
    u.y = *reinterpret_cast<unsigned*>(&hi);
    *p = u;
  }
}
}  // namespace

// row_map null: row t of the output; else row row_map[t] (below max_rows; a negative entry is skipped).
FMX_EXPORT int fmx_rmsnorm_rows(const void* x, long long x_stride, int x_dtype, const float* w, float eps, void* out,
                                long long out_stride, int out_dtype, const long long* row_map, long long max_rows, int rows,
                                int n, int* status, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rows < 0 || n <= 0 || x_stride < n || out_stride < n) return fmx_fail("fmx_rmsnorm_rows: bad sizes rows=%d n=%d", rows, n);
#define FMX_NR(TI, TO)                                                                                                  \
  fmx_launch(rmsnorm_rows_kernel<TI, TO>, dim3(rows), dim3(NORM_BLOCK), 0, stream, (const TI*)x, x_stride, w, eps, (TO*)out, \
             out_stride, row_map, max_rows, n, status)
  if (x_dtype == FMX_F32 && out_dtype == FMX_F32) FMX_NR(float, float);
  else if (x_dtype == FMX_F32 && out_dtype == FMX_BF16) FMX_NR(float, bf16);
  else if (x_dtype == FMX_BF16 && out_dtype == FMX_BF16) FMX_NR(bf16, bf16);
  else if (x_dtype == FMX_BF16 && out_dtype == FMX_F32) FMX_NR(bf16, float);
  else return fmx_fail("fmx_rmsnorm_rows: unknown dtypes %d, %d", x_dtype, out_dtype);
#undef FMX_NR
  FMX_LAUNCH_CHECK();
  return 0;
}

FMX_EXPORT int fmx_sigmoid_gate(void* o, long long o_stride, int o_dtype, const void* g, long long g_stride, int g_dtype,
                                int rows, int cols, int group, cudaStream_t stream) {
  if (rows == 0 || cols == 0) return 0;
  if (rows < 0 || cols < 0 || group <= 0 || o_stride < cols) return fmx_fail("fmx_sigmoid_gate: bad sizes rows=%d cols=%d group=%d", rows, cols, group);
  const bool vec = o_dtype == FMX_BF16 && g_dtype == FMX_F32 && cols % 4 == 0 && o_stride % 4 == 0 && ((uintptr_t)o & 7) == 0 &&
                   (group == 1 ? (g_stride % 4 == 0 && ((uintptr_t)g & 15) == 0) : group % 4 == 0);
  const long long n = (long long)rows * (vec ? cols / 4 : cols), cap = (long long)fmx_num_sms() * 16;
  const int block = 256;
  const int grid = (int)((n + block - 1) / block < cap ? (n + block - 1) / block : cap);
  if (vec) {
    fmx_launch(sigmoid_gate_vec_kernel, dim3(grid), dim3(block), 0, stream, (bf16*)o, o_stride, (const float*)g, g_stride,
               (long long)rows, cols, group);
    FMX_LAUNCH_CHECK();
    return 0;
  }
#define FMX_SG(TO, TG)                                                                                                \
  fmx_launch(sigmoid_gate_kernel<TO, TG>, dim3(grid), dim3(block), 0, stream, (TO*)o, o_stride, (const TG*)g, g_stride, \
             (long long)rows, cols, group)
  if (o_dtype == FMX_F32 && g_dtype == FMX_F32) FMX_SG(float, float);
  else if (o_dtype == FMX_BF16 && g_dtype == FMX_F32) FMX_SG(bf16, float);
  else if (o_dtype == FMX_BF16 && g_dtype == FMX_BF16) FMX_SG(bf16, bf16);
  else return fmx_fail("fmx_sigmoid_gate: unknown dtypes %d, %d", o_dtype, g_dtype);
#undef FMX_SG
  FMX_LAUNCH_CHECK();
  return 0;
}

// a and b: rows of n values of type in_dtype; out of type out_dtype.
FMX_EXPORT int fmx_rmsnorm_pair_mean(const void* a, long long a_stride, const void* b, long long b_stride, int in_dtype,
                                     const float* wa, const float* wb, float eps, void* out, long long out_stride, int out_dtype,
                                     int rows, int n, cudaStream_t stream) {
  if (rows == 0) return 0;
  if (rows < 0 || n <= 0 || a_stride < n || b_stride < n || out_stride < n)
    return fmx_fail("fmx_rmsnorm_pair_mean: bad sizes rows=%d n=%d", rows, n);
#define FMX_PM(TI, TO)                                                                                                   \
  fmx_launch(rmsnorm_pair_mean_kernel<TI, TO>, dim3(rows), dim3(NORM_BLOCK), 0, stream, (const TI*)a, a_stride, (const TI*)b, \
             b_stride, wa, wb, eps, (TO*)out, out_stride, n)
  if (in_dtype == FMX_F32 && out_dtype == FMX_F32) FMX_PM(float, float);
  else if (in_dtype == FMX_F32 && out_dtype == FMX_BF16) FMX_PM(float, bf16);
  else if (in_dtype == FMX_BF16 && out_dtype == FMX_BF16) FMX_PM(bf16, bf16);
  else if (in_dtype == FMX_BF16 && out_dtype == FMX_F32) FMX_PM(bf16, float);
  else return fmx_fail("fmx_rmsnorm_pair_mean: unknown dtypes %d, %d", in_dtype, out_dtype);
#undef FMX_PM
  FMX_LAUNCH_CHECK();
  return 0;
}
