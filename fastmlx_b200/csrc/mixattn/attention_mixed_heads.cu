// Tiled paged attention with sigmoid weights that are mixed across heads, for a bfloat16 cache.
//
// A query at position p of head g gives a visible key j the weight w_g(p, j) = sigmoid(cap(scale q_g . k_kv(g)(j)) + b_g);
// the heads' weights are mixed, w'_h = sum_g M[h, g] w_g, and head h applies w'_h to the values of its own key/value
// head.  Mixing needs the weights of every head for one (query, key) pair in one place, so a block owns ALL heads of a
// tile of up to TQ consecutive tokens of one request and walks the keys in tiles of 32, aligned to absolute positions:
//
//   load      the tile's keys and values of every key/value head into shared memory (16-byte copies; rows out of
//             sight are zeros);
//   scores    a warp takes a unit (token i, key/value head c): lane = key, the dot products of the unit's query heads
//             with the lane's key in 32-bit (a key's 8 values are fetched once for all heads of the unit), scale, cap,
//             sigmoid -> P[i, g, key] in shared memory;
//   mix       the same warp, for its unit's heads h: W[i, h, key] = sum_g M[h, g] P[i, g, key], g in order;
//   values    the same warp: lane = a run of FMX_VPL value dimensions; acc[h] += W[i, h, key] v_c(key), key by key,
//             one fetch of a value row for all heads of the unit.  The accumulators stay in registers over all tiles.
//
// Queries are 32-bit, keys and values are exact in 32-bit, and every sum is made of 32-bit multiply-adds in an order that
// the indices alone fix (over heads and over keys one chain in index order; a dot product two chains, over the even and
// the odd runs of eight dimensions): no tensor cores, because a weight that is a 32-bit sum of
// 32-bit sigmoids has no two-term bfloat16 form that the mix would keep.  Nothing is normalised over the keys, so a
// token's keys may be shared out over `splits` blocks whose partial outputs a second kernel adds up in split order.
//
// One library per (FMX_VPL, FMX_PER): FMX_VPL value dimensions per lane (values up to 32 * FMX_VPL wide), FMX_PER query
// heads per key/value head at most.  US units per warp: 1 (single tokens) or USP (portions: at most FMX_USP_MAX, so that two
// blocks of eight warps fit a multiprocessor's registers; sixteen warps where shared memory leaves room for one block only).
#include <math.h>
#include "common.cuh"

#ifndef FMX_VPL
#define FMX_VPL 2
#endif
#ifndef FMX_USP_MAX
#define FMX_USP_MAX 2
#endif
#ifndef FMX_PER
#define FMX_PER 4
#endif

namespace {
constexpr int VPL = FMX_VPL, PER = FMX_PER;
constexpr int WARPS = 8, TK = 32;
constexpr int USP_MAX = FMX_USP_MAX;
constexpr int USP = (64 / (VPL * PER)) < 1 ? 1 : ((64 / (VPL * PER)) > USP_MAX ? USP_MAX : (64 / (VPL * PER)));
constexpr int VROW = 32 * VPL + 8;                // a value row in shared memory: padded to the lanes' runs, plus 16 bytes
constexpr size_t SMEM_LIMIT = 220 * 1024;

__device__ __forceinline__ void load8(const bf16* p, float* f) {       // 16 bytes -> 8 floats
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(h[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}

template <int N> __device__ __forceinline__ void load_run(const bf16* p, float* f) {      // N = 1, 2, 4 or 8 values
  if constexpr (N == 1) {
    f[0] = __bfloat162float(p[0]);
  } else if constexpr (N == 2) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    f[0] = x.x; f[1] = x.y;
  } else if constexpr (N == 4) {
    const uint2 u = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
    const float2 a = __bfloat1622float2(h[0]), b = __bfloat1622float2(h[1]);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
  } else {
    load8(p, f);
  }
}

struct Layout {             // offsets into dynamic shared memory, in bytes, every region on 16 bytes
  size_t q, m, hb, p, w, k, v, total;
  int kst;                  // elements of a key row
};
__host__ __device__ inline size_t up16(size_t x) { return (x + 15) / 16 * 16; }
__host__ __device__ inline Layout layout_for(int TQ, int nh, int nkv, int hd) {
  Layout L;
  L.kst = (hd + 7) / 8 * 8 + 8;
  size_t at = 0;
  L.q = at; at += up16((size_t)TQ * nh * hd * 4);
  L.m = at; at += up16((size_t)nh * nh * 4);
  L.hb = at; at += up16((size_t)nh * 4);
  L.p = at; at += up16((size_t)TQ * nh * TK * 4);
  L.w = at; at += up16((size_t)TQ * nh * TK * 4);
  L.k = at; at += up16((size_t)nkv * TK * L.kst * 2);
  L.v = at; at += up16((size_t)nkv * TK * VROW * 2);
  L.total = at;
  return L;
}

template <int US, int NW>
__global__ void __launch_bounds__(NW * 32)
mixed_heads_attention_kernel(const float* q, long long q_stride, const bf16* kv, const int* block_tables, int bt_stride,
                             const int* token_row, const int* positions, const int* row_start, float* part, bf16* out,
                             long long out_stride, int n_tokens, int nh, int nkv, int hd, int vd, int page_size,
                             long long num_pages, float scale, float softcap, int window, int R,
                             const float* __restrict__ head_bias, const float* __restrict__ mix, int TQ, int splits,
                             int* status) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  pdl_wait();
  pdl_trigger();
  const int t0 = n_tokens - 1 - (int)blockIdx.x, split = blockIdx.y;      // a row's last tiles walk the most keys: they start first
  const int row = token_row[t0];
  if (row < 0 || row >= R) {
    if (threadIdx.x == 0) fmx_set_status(status, FMX_BAD_ROW, row, t0);
    return;
  }
  const int first = row_start[row];
  if ((t0 - first) % TQ != 0) return;                 // another block's tile holds this token
  const int n_q = min(TQ, row_start[row + 1] - t0);
  const int per = nh / nkv;
  const Layout L = layout_for(TQ, nh, nkv, hd);
  float* qs = reinterpret_cast<float*>(smem_raw + L.q);
  float* Ms = reinterpret_cast<float*>(smem_raw + L.m);
  float* hbs = reinterpret_cast<float*>(smem_raw + L.hb);
  float* Ps = reinterpret_cast<float*>(smem_raw + L.p);
  float* Ws = reinterpret_cast<float*>(smem_raw + L.w);
  bf16* Ks = reinterpret_cast<bf16*>(smem_raw + L.k);
  bf16* Vs = reinterpret_cast<bf16*>(smem_raw + L.v);
  const int KST = L.kst;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  for (int x = threadIdx.x; x < n_q * nh * hd; x += blockDim.x) {
    const int i = x / (nh * hd);
    qs[x] = q[(long long)(t0 + i) * q_stride + (x - i * nh * hd)];
  }
  for (int x = threadIdx.x; x < nh * nh; x += blockDim.x) Ms[x] = mix[x];
  for (int x = threadIdx.x; x < nh; x += blockDim.x) hbs[x] = head_bias != nullptr ? head_bias[x] : 0.f;
  for (int x = threadIdx.x; x < nkv * TK * VROW; x += blockDim.x) Vs[x] = __float2bfloat16_rn(0.f);   // the rows' padding stays zero

  const int pos0 = positions[t0], pos_last = positions[t0 + n_q - 1];
  const int lo_min = window > 0 ? max(0, pos0 - window + 1) : 0;
  float acc[US][PER][VPL];
#pragma unroll
  for (int s = 0; s < US; ++s)
#pragma unroll
    for (int hh = 0; hh < PER; ++hh)
#pragma unroll
      for (int k = 0; k < VPL; ++k) acc[s][hh][k] = 0.f;

  int kt_first = lo_min / TK, kt_end = pos_last >= 0 ? pos_last / TK + 1 : 0;      // a padding row (position -1) walks nothing
  if (splits > 1) {
    const int n = max(0, kt_end - kt_first), chunk = (n + splits - 1) / splits;
    kt_first = kt_first + split * chunk;
    kt_end = min(kt_end, kt_first + chunk);
  }
  const long long plane = (long long)nkv * page_size * hd;
  const long long page_elems = (long long)nkv * page_size * (hd + vd);
  const int* bt = block_tables + (long long)row * bt_stride;
  const float inv_cap = softcap > 0.f ? 1.0f / softcap : 0.f;
  const bool kvec = (hd & 7) == 0 && (vd & 7) == 0;

  // the warp's units: (token of the tile, key/value head), the same for every tile of keys
  int u_i[US], u_c[US];
  bool u_on[US];
#pragma unroll
  for (int s = 0; s < US; ++s) {
    const int n = warp + NW * s;
    u_on[s] = n < n_q * nkv;
    u_i[s] = u_on[s] ? n / nkv : 0;
    u_c[s] = u_on[s] ? n - u_i[s] * nkv : 0;
  }
  // rows of a tile are copied by groups of lanes: `lpr` lanes (a power of two) take a row's 16-byte pieces
  const int kc = hd / 8, vc = vd / 8, cpr = kc + vc;
  int lpr_log = 0;
  while ((1 << lpr_log) < cpr) ++lpr_log;
  const int lpr = 1 << lpr_log;                                      // lanes per row
  const int page_log = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;

  for (int kt = kt_first; kt < kt_end; ++kt) {
    __syncthreads();                                    // the tile before is done with K, V and P (and q, M are written)
    // ---- load: rows (c, jj) of keys and of values
    if (kvec) {
      // 16-byte asynchronous copies, all of a thread's in flight together; a row out of sight is filled with zeros.
      // A thread owns (key of the tile, 16-byte piece of a row) pairs: it looks the key's page up once and then walks
      // the key/value heads, whose rows lie a fixed distance apart in the page and in shared memory
      for (int idx = threadIdx.x; idx < (TK << lpr_log); idx += blockDim.x) {
        const int jj = idx >> lpr_log, ch = idx & (lpr - 1);
        if (ch >= cpr) continue;
        const int j = kt * TK + jj;
        const bf16* src = kv;
        unsigned bytes = 0;
        long long step = 0;
        const bool is_k = ch < kc;
        if (j >= lo_min && j <= pos_last) {
          const int blk = page_log >= 0 ? j >> page_log : j / page_size;
          const int page = blk < bt_stride ? bt[blk] : -1;
          if (page < 0 || page >= num_pages) {
            fmx_set_status(status, FMX_BAD_PAGE, page, t0);
          } else {
            const int at = j - blk * page_size;
            src = is_k ? kv + (long long)page * page_elems + (long long)at * hd + ch * 8
                       : kv + (long long)page * page_elems + plane + (long long)at * vd + (ch - kc) * 8;
            step = (long long)page_size * (is_k ? hd : vd);
            bytes = 16;
          }
        }
        unsigned sa = (unsigned)__cvta_generic_to_shared(is_k ? Ks + (long long)jj * KST + ch * 8 : Vs + (long long)jj * VROW + (ch - kc) * 8);
        const unsigned sstep = (unsigned)(TK * (is_k ? KST : VROW) * 2);
        for (int c = 0; c < nkv; ++c) {
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(sa), "l"(src), "r"(bytes));
          sa += sstep;
          src += step;
        }
      }
      asm volatile("cp.async.commit_group;\n" ::);
      asm volatile("cp.async.wait_group 0;\n" ::);
    } else {
      for (int x = threadIdx.x; x < nkv * TK * (hd + vd); x += blockDim.x) {
        const int r = x / (hd + vd), e = x - r * (hd + vd);
        const int c = r / TK, jj = r - c * TK;
        const int j = kt * TK + jj;
        bf16 val = __float2bfloat16_rn(0.f);
        if (j >= lo_min && j <= pos_last) {
          const int blk = j / page_size;
          const int page = blk < bt_stride ? bt[blk] : -1;
          if (page < 0 || page >= num_pages) {
            fmx_set_status(status, FMX_BAD_PAGE, page, t0);
          } else {
            const long long at = (long long)c * page_size + (j - blk * page_size);
            val = e < hd ? kv[(long long)page * page_elems + at * hd + e]
                         : kv[(long long)page * page_elems + plane + at * vd + (e - hd)];
          }
        }
        if (e < hd) Ks[(long long)r * KST + e] = val;
        else Vs[(long long)r * VROW + (e - hd)] = val;
      }
    }
    __syncthreads();
    // ---- scores: P[i, h, key]; the units of a warp side by side, so that their chains of multiply-adds interleave
    {
      float dot[US][PER], dot2[US][PER];                  // a dot product as two chains: even and odd runs of eight dimensions
#pragma unroll
      for (int s = 0; s < US; ++s)
#pragma unroll
        for (int hh = 0; hh < PER; ++hh) dot[s][hh] = dot2[s][hh] = 0.f;
      if ((hd & 7) == 0) {
        auto run = [&](int e, float (&into)[US][PER]) {
#pragma unroll
          for (int s = 0; s < US; ++s) {
            if (!u_on[s]) continue;
            float kf[8];
            load8(Ks + ((long long)u_c[s] * TK + lane) * KST + e, kf);
            const float* qb = qs + ((long long)u_i[s] * nh + (long long)u_c[s] * per) * hd + e;
#pragma unroll
            for (int hh = 0; hh < PER; ++hh) {
              if (hh < per) {
                const float4 a = *reinterpret_cast<const float4*>(qb + (long long)hh * hd);
                const float4 b = *reinterpret_cast<const float4*>(qb + (long long)hh * hd + 4);
                float d = into[s][hh];
                d = fmaf(a.x, kf[0], d); d = fmaf(a.y, kf[1], d); d = fmaf(a.z, kf[2], d); d = fmaf(a.w, kf[3], d);
                d = fmaf(b.x, kf[4], d); d = fmaf(b.y, kf[5], d); d = fmaf(b.z, kf[6], d); d = fmaf(b.w, kf[7], d);
                into[s][hh] = d;
              }
            }
          }
        };
        int e = 0;
        for (; e + 16 <= hd; e += 16) {
          run(e, dot);
          run(e + 8, dot2);
        }
        if (e < hd) run(e, dot);
#pragma unroll
        for (int s = 0; s < US; ++s)
#pragma unroll
          for (int hh = 0; hh < PER; ++hh) dot[s][hh] += dot2[s][hh];
      } else {
        for (int e = 0; e < hd; ++e) {
#pragma unroll
          for (int s = 0; s < US; ++s) {
            if (!u_on[s]) continue;
            const float kf = __bfloat162float(Ks[((long long)u_c[s] * TK + lane) * KST + e]);
            const float* qb = qs + ((long long)u_i[s] * nh + (long long)u_c[s] * per) * hd + e;
#pragma unroll
            for (int hh = 0; hh < PER; ++hh)
              if (hh < per) dot[s][hh] = fmaf(qb[(long long)hh * hd], kf, dot[s][hh]);
          }
        }
      }
      const int j = kt * TK + lane;
#pragma unroll
      for (int s = 0; s < US; ++s) {
        if (!u_on[s]) continue;
        const int pos_i = pos0 + u_i[s];
        const int lo_i = window > 0 ? max(0, pos_i - window + 1) : 0;
        const bool valid = j >= lo_i && j <= pos_i;
#pragma unroll
        for (int hh = 0; hh < PER; ++hh) {
          if (hh < per) {
            const int h = u_c[s] * per + hh;
            float sc = dot[s][hh] * scale;
            if (softcap > 0.f) sc = softcap * tanhf(sc * inv_cap);
            Ps[((long long)u_i[s] * nh + h) * TK + lane] = valid ? __fdividef(1.0f, 1.0f + __expf(-(sc + hbs[h]))) : 0.f;
          }
        }
      }
    }
    __syncthreads();
    // ---- mix: W[i, h, key] for the heads of the warp's units
    {
      float wm[US][PER];
#pragma unroll
      for (int s = 0; s < US; ++s)
#pragma unroll
        for (int hh = 0; hh < PER; ++hh) wm[s][hh] = 0.f;
      if ((nh & 3) == 0) {
#pragma unroll 2
        for (int g = 0; g < nh; g += 4) {               // four heads' weights and four values of a row of the mix at a time
#pragma unroll
          for (int s = 0; s < US; ++s) {
            if (!u_on[s]) continue;
            const float* pi = Ps + ((long long)u_i[s] * nh + g) * TK + lane;
            const float p0 = pi[0], p1 = pi[TK], p2 = pi[2 * TK], p3 = pi[3 * TK];
#pragma unroll
            for (int hh = 0; hh < PER; ++hh) {
              if (hh < per) {
                const float4 m4 = *reinterpret_cast<const float4*>(Ms + (u_c[s] * per + hh) * nh + g);
                float w = wm[s][hh];
                w = fmaf(m4.x, p0, w); w = fmaf(m4.y, p1, w); w = fmaf(m4.z, p2, w); w = fmaf(m4.w, p3, w);
                wm[s][hh] = w;
              }
            }
          }
        }
      } else {
        for (int g = 0; g < nh; ++g) {
#pragma unroll
          for (int s = 0; s < US; ++s) {
            if (!u_on[s]) continue;
            const float pv = Ps[((long long)u_i[s] * nh + g) * TK + lane];
#pragma unroll
            for (int hh = 0; hh < PER; ++hh)
              if (hh < per) wm[s][hh] = fmaf(Ms[(u_c[s] * per + hh) * nh + g], pv, wm[s][hh]);
          }
        }
      }
#pragma unroll
      for (int s = 0; s < US; ++s) {
        if (!u_on[s]) continue;
#pragma unroll
        for (int hh = 0; hh < PER; ++hh)
          if (hh < per) Ws[((long long)u_i[s] * nh + (long long)u_c[s] * per + hh) * TK + lane] = wm[s][hh];
      }
    }
    __syncwarp();
    // ---- values: the warp's own rows of W meet the values, four keys at a time
#pragma unroll 2
    for (int jj = 0; jj < TK; jj += 4) {
#pragma unroll
      for (int s = 0; s < US; ++s) {
        if (!u_on[s]) continue;
        const float* wrow = Ws + ((long long)u_i[s] * nh + (long long)u_c[s] * per) * TK + jj;
        const bf16* vb = Vs + ((long long)u_c[s] * TK + jj) * VROW + lane * VPL;
        float4 w4[PER];
#pragma unroll
        for (int hh = 0; hh < PER; ++hh)
          w4[hh] = hh < per ? *reinterpret_cast<const float4*>(wrow + hh * TK) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          float v[VPL];
          load_run<VPL>(vb + (long long)x * VROW, v);
#pragma unroll
          for (int hh = 0; hh < PER; ++hh) {
            const float w = x == 0 ? w4[hh].x : x == 1 ? w4[hh].y : x == 2 ? w4[hh].z : w4[hh].w;
#pragma unroll
            for (int k = 0; k < VPL; ++k) acc[s][hh][k] = fmaf(w, v[k], acc[s][hh][k]);
          }
        }
      }
    }
    __syncwarp();
  }
  // ---- out
#pragma unroll
  for (int s = 0; s < US; ++s) {
    if (!u_on[s]) continue;
    const int i = u_i[s], c = u_c[s];
#pragma unroll
    for (int hh = 0; hh < PER; ++hh) {
      if (hh >= per) continue;
      const int h = c * per + hh;
#pragma unroll
      for (int k = 0; k < VPL; ++k) {
        const int e = lane * VPL + k;
        if (e >= vd) continue;
        if (splits > 1) part[((long long)split * n_tokens + t0 + i) * nh * vd + (long long)h * vd + e] = acc[s][hh][k];
        else out[(long long)(t0 + i) * out_stride + (long long)h * vd + e] = __float2bfloat16_rn(acc[s][hh][k]);
      }
    }
  }
}

__global__ void mixed_heads_combine_kernel(const float* part, bf16* out, long long out_stride, int n_tokens, int width, int splits) {
  pdl_wait();
  pdl_trigger();
  const long long n = (long long)n_tokens * width;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < n; idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / width;
    const int x = (int)(idx - t * width);
    float s = 0.f;
    for (int k = 0; k < splits; ++k) s += part[(long long)k * n + idx];
    out[t * out_stride + x] = __float2bfloat16_rn(s);
  }
}

// Tokens per tile, units per warp and warps per block for a step whose longest row brings max_q_len tokens; 0: the sizes
// do not fit.  Portions run 8 warps where two blocks fit a multiprocessor's shared memory, else 16 warps in one block.
int plan_tile(int nh, int nkv, int hd, int vd, int max_q_len, int* us_out, int* nw_out) {
  if (nh <= 0 || nkv <= 0 || nh % nkv || nh / nkv > PER || vd > 32 * VPL || hd <= 0) return 0;
  int nw = WARPS;
  const int need = (nkv + nw - 1) / nw;                 // units per warp that one token needs
  int us = max_q_len > 1 ? USP : 1;
  if (need > us) us = USP;
  if (need > us) return 0;
  auto tokens = [&](int warps) {
    int t = (warps * us) / nkv;
    if (t < 1) t = 1;
    if (t > max_q_len) t = max_q_len > 0 ? max_q_len : 1;
    while (t > 1 && layout_for(t, nh, nkv, hd).total > SMEM_LIMIT) --t;
    return t;
  };
  int tq = tokens(nw);
  if (layout_for(tq, nh, nkv, hd).total > SMEM_LIMIT) return 0;
  if (max_q_len > 1 && 2 * layout_for(tq, nh, nkv, hd).total + 4096 > 227 * 1024) {
    const int tq16 = tokens(2 * WARPS);                 // one block per multiprocessor either way: twice the warps
    if (tq16 * nkv > WARPS * us) { nw = 2 * WARPS; tq = tq16; }
  }
  if (us == USP && USP > 1 && (tq * nkv + nw - 1) / nw <= 1) us = 1;
  *us_out = us;
  *nw_out = nw;
  return tq;
}
}  // namespace

FMX_EXPORT int fmx_mixattn_vpl() { return VPL; }
FMX_EXPORT int fmx_mixattn_per() { return PER; }

// How many blocks a token's keys should be shared out over (1 for portions), or 0 where the kernel does not take
// the sizes (the caller then uses the kernel with one warp per token and head).
FMX_EXPORT int fmx_mixattn_plan(int n_tokens, int nh, int nkv, int hd, int vd, int max_q_len, int max_ctx) {
  int us = 1, nw = WARPS;
  if (plan_tile(nh, nkv, hd, vd, max_q_len, &us, &nw) == 0) return 0;
  if (max_q_len > 1 || n_tokens <= 0) return 1;
  const int tiles = (max_ctx + TK - 1) / TK;
  // as many blocks as are resident at once (two per multiprocessor where their shared memory allows), no more: a
  // second round of a few blocks would double the time
  const size_t smem = layout_for(1, nh, nkv, hd).total;
  const int slots = fmx_num_sms() * (2 * smem + 4096 <= 227 * 1024 ? 2 : 1);
  int splits = slots / n_tokens;
  if (splits > tiles / 2) splits = tiles / 2;           // at least two tiles of keys per block
  if (splits > 32) splits = 32;
  return splits < 1 ? 1 : splits;
}

// q [T, nh*hd] 32-bit; kv: bfloat16 pages of [nkv, page, hd] keys and [nkv, page, vd] values; out [T, nh*vd] bfloat16
// in rows of out_stride; part: splits * T * nh * vd floats where splits > 1; mix [nh, nh] and head_bias [nh] (or null)
// 32-bit.  row_start [R + 1]: where each row's tokens start in the step.
FMX_EXPORT int fmx_mixattn(const float* q, long long q_stride, const void* kv, const int* block_tables, int bt_stride,
                           const int* token_row, const int* positions, const int* row_start, float* part, void* out,
                           long long out_stride, int n_tokens, int nh, int nkv, int hd, int vd, int page_size,
                           long long num_pages, float scale, float softcap, int window, int R, const float* head_bias,
                           const float* mix, int max_q_len, int splits, int* status, cudaStream_t stream) {
  if (n_tokens == 0) return 0;
  if (n_tokens < 0 || page_size <= 0 || window < 0 || splits < 1 || (splits > 1 && part == nullptr) || mix == nullptr)
    return fmx_fail("fmx_mixattn: bad sizes T=%d page=%d window=%d splits=%d", n_tokens, page_size, window, splits);
  if (out_stride < (long long)nh * vd) return fmx_fail("fmx_mixattn: output rows too narrow");
  int us = 1, nw = WARPS;
  const int tq = plan_tile(nh, nkv, hd, vd, max_q_len, &us, &nw);
  if (tq == 0) return fmx_fail("fmx_mixattn: sizes nh=%d nkv=%d hd=%d vd=%d do not fit this library (%d values per lane, %d heads per key head)",
                               nh, nkv, hd, vd, VPL, PER);
  if (((uintptr_t)q & 15) || (q_stride & 3) || ((nh * hd) & 3)) return fmx_fail("fmx_mixattn: queries must lie on 16 bytes");
  const Layout L = layout_for(tq, nh, nkv, hd);
  const dim3 grid(n_tokens, splits);
  auto launch = [&](auto kernel) {
    static thread_local void* raised = nullptr;
    if (L.total > 48 * 1024 && raised != (void*)kernel) {
      if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_LIMIT) != cudaSuccess) return 1;
      raised = (void*)kernel;
    }
    fmx_launch(kernel, grid, dim3(nw * 32), L.total, stream, q, q_stride, (const bf16*)kv, block_tables, bt_stride, token_row,
               positions, row_start, part, (bf16*)out, out_stride, n_tokens, nh, nkv, hd, vd, page_size, num_pages, scale,
               softcap, window, R, head_bias, mix, tq, splits, status);
    return 0;
  };
  int rc;
  if (us == 1 && nw == WARPS) rc = launch(mixed_heads_attention_kernel<1, WARPS>);
  else if (us == 1) rc = launch(mixed_heads_attention_kernel<1, 2 * WARPS>);
  else if (nw == WARPS) rc = launch(mixed_heads_attention_kernel<USP, WARPS>);
  else rc = launch(mixed_heads_attention_kernel<USP, 2 * WARPS>);
  if (rc) return fmx_fail("fmx_mixattn: the kernel's shared memory could not be raised");
  FMX_LAUNCH_CHECK();
  if (splits > 1) {
    const long long n = (long long)n_tokens * nh * vd;
    const int blocks = (int)((n + 255) / 256 < 4096 ? (n + 255) / 256 : 4096);
    fmx_launch(mixed_heads_combine_kernel, dim3(blocks), dim3(256), 0, stream, (const float*)part, (bf16*)out, out_stride, n_tokens,
               nh * vd, splits);
    FMX_LAUNCH_CHECK();
  }
  return 0;
}
