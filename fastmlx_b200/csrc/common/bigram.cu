// Token embedding with a hashed bigram table added to it.
//
// out[t] = E[id_t] + B[(id_(t-1) * mul_prev + id_t * mul_cur) mod buckets], summed in 32-bit and left in 32-bit:
// the sum is the residual stream's first value.  A request's first token (position 0) takes row `buckets`, the
// table's last.  The token before a row's first token of this step is one integer of per-request state,
// state[slot]: the block of the row's first token reads it and then replaces it by the row's last token, so that
// no other block touches the slot.  A row whose slot is -1 (the padding rows of a captured step) or whose position
// is negative gets zeros and leaves no state.
#include "common.cuh"

namespace {
template <typename T>
__global__ void __launch_bounds__(128)
embed_bigram_kernel(const int* ids, const T* __restrict__ table, const T* __restrict__ bigram, const int* positions,
                    const int* token_row, const int* row_start, const int* row_slot, int* state, long long state_stride,
                    float* out, int d, long long vocab, long long buckets, long long mul_prev, long long mul_cur, int R,
                    int max_slots, int* status) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x;
  float* dst = out + (long long)t * d;
  const int r = token_row[t];
  const int slot = (r >= 0 && r < R) ? row_slot[r] : -1;
  const int pos = positions[t];
  const long long id = ids[t];
  bool ok = slot >= 0 && slot < max_slots && pos >= 0;
  if (r < 0 || r >= R) { if (threadIdx.x == 0) fmx_set_status(status, FMX_BAD_ROW, r, t); }
  else if (slot >= max_slots) { if (threadIdx.x == 0) fmx_set_status(status, FMX_BAD_SLOT, slot, t); }
  else if (ok && (id < 0 || id >= vocab)) {
    if (threadIdx.x == 0) fmx_set_status(status, FMX_BAD_TOKEN, id, t);
    ok = false;
  }
  if (!ok) {
    for (int e = threadIdx.x; e < d; e += blockDim.x) dst[e] = 0.f;
    return;
  }
  const int first = row_start[r];
  long long prev;
  if (t == first) {
    // every thread reads the old value; one thread replaces it after all have read
    prev = state[(long long)slot * state_stride];
    __syncthreads();
    if (threadIdx.x == 0) state[(long long)slot * state_stride] = ids[row_start[r + 1] - 1];
  } else {
    prev = ids[t - 1];
  }
  long long brow = buckets;
  if (pos > 0) {
    brow = (prev * mul_prev + id * mul_cur) % buckets;
    if (brow < 0) brow += buckets;
  }
  const T* e_row = table + id * d;
  const T* b_row = bigram + brow * d;
  for (int e = threadIdx.x; e < d; e += blockDim.x) dst[e] = to_f(e_row[e]) + to_f(b_row[e]);
}
}  // namespace

// table [vocab, d] and bigram [buckets + 1, d] of `dtype`; state: int32, one value per slot in rows of state_stride.
FMX_EXPORT int fmx_embed_bigram(const int* ids, const void* table, const void* bigram, const int* positions,
                                const int* token_row, const int* row_start, const int* row_slot, int* state,
                                long long state_stride, float* out, int T, int d, long long vocab, long long buckets,
                                long long mul_prev, long long mul_cur, int R, int max_slots, int dtype, int* status,
                                cudaStream_t stream) {
  if (T == 0) return 0;
  if (T < 0 || d <= 0 || vocab <= 0 || buckets <= 0 || R <= 0 || max_slots <= 0 || state_stride < 1)
    return fmx_fail("fmx_embed_bigram: bad sizes T=%d d=%d vocab=%lld buckets=%lld R=%d", T, d, vocab, buckets, R);
  if (dtype == FMX_F32)
    fmx_launch(embed_bigram_kernel<float>, dim3(T), dim3(128), 0, stream, ids, (const float*)table, (const float*)bigram,
               positions, token_row, row_start, row_slot, state, state_stride, out, d, vocab, buckets, mul_prev, mul_cur, R,
               max_slots, status);
  else if (dtype == FMX_BF16)
    fmx_launch(embed_bigram_kernel<bf16>, dim3(T), dim3(128), 0, stream, ids, (const bf16*)table, (const bf16*)bigram,
               positions, token_row, row_start, row_slot, state, state_stride, out, d, vocab, buckets, mul_prev, mul_cur, R,
               max_slots, status);
  else
    return fmx_fail("fmx_embed_bigram: unknown dtype %d", dtype);
  FMX_LAUNCH_CHECK();
  return 0;
}
