// The steps on either side of the attention / MoE hot path: rms_norm (with
// optional residual add), rotary position embedding, and fill_kv_cache.  All
// three are HBM-bound row kernels: 128-bit coalesced accesses, fp32 reductions
// through warp shuffles, one rounding per store.
//
// Reference semantics
//   rms_norm        python/dlBLAS/dlblas/kernels/rms_norm.py:8-132
//                     new_x = x + residual (storage dtype); out = (w * new_x_f32 * rsqrt(mean(x^2)+eps)) -> dtype
//   add_rms_norm    python/dlBLAS/dlblas/kernels/add_rms_norm.py:11-80
//                     same, but out = (new_x_f32 * rsqrt(..)) -> dtype, then * w in the storage dtype
//   apply_rotary    python/dlBLAS/dlblas/kernels/apply_rotary_pos_emb.py:8-164
//                     lo' = lo*cos_lo - hi*sin_lo ; hi' = hi*cos_hi + lo*sin_hi, arithmetic in q's dtype
//   fill_kv_cache   python/dlBLAS/dlblas/kernels/fill_kv_cache.py:24-185
//                     new tokens of each sequence go to slot (history + i) % page of page
//                     block_offsets[b, (history + i) / page]
#include <type_traits>

#include "common.cuh"

namespace dlb {

// ----------------------------------------------------------------------------
// rms_norm
// ----------------------------------------------------------------------------
__device__ __forceinline__ float block_sum_256(float v, float* red) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = (lane < (int)(blockDim.x >> 5)) ? red[lane] : 0.f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
  return t;   // every thread holds the block total
}

// Vector path: 256 threads, VPT 16-byte vectors per thread kept in registers between the two passes.
template <typename T, int VPT>
__global__ void __launch_bounds__(256) rms_norm_vec_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                           const T* __restrict__ res, T* __restrict__ out,
                                                           T* __restrict__ out_res, int n, int64_t xs, int64_t rs,
                                                           int64_t os, float eps, int weight_after_cast) {
  using T2 = typename Elem<T>::T2;
  __shared__ float red[8];
  const int64_t row = blockIdx.x;
  const int nvec = n >> 3;
  const uint4* xp = reinterpret_cast<const uint4*>(x + row * xs);
  const uint4* rp = res ? reinterpret_cast<const uint4*>(res + row * rs) : nullptr;
  uint4* orp = out_res ? reinterpret_cast<uint4*>(out_res + row * rs) : nullptr;
  uint4 v[VPT];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < nvec) {
      v[i] = __ldg(xp + c);
      if (rp) {
        const uint4 r = __ldg(rp + c);
        T2* a = reinterpret_cast<T2*>(&v[i]);
        const T2* b = reinterpret_cast<const T2*>(&r);
#pragma unroll
        for (int j = 0; j < 4; ++j) {   // the add happens in the storage dtype, as in the reference
          const float2 fa = Elem<T>::to_f2(a[j]), fb = Elem<T>::to_f2(b[j]);
          a[j] = Elem<T>::from_f2(fa.x + fb.x, fa.y + fb.y);
        }
        if (orp) orp[c] = v[i];
      }
      const T2* a = reinterpret_cast<const T2*>(&v[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = Elem<T>::to_f2(a[j]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
  }
  const float inv = rsqrtf(block_sum_256(ss, red) * (1.0f / n) + eps);
  const uint4* wp = reinterpret_cast<const uint4*>(w);
  uint4* op = reinterpret_cast<uint4*>(out + row * os);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = threadIdx.x + i * 256;
    if (c < nvec) {
      const uint4 wv = __ldg(wp + c);
      const T2* a = reinterpret_cast<const T2*>(&v[i]);
      const T2* b = reinterpret_cast<const T2*>(&wv);
      uint4 o;
      T2* o2 = reinterpret_cast<T2*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = Elem<T>::to_f2(a[j]), g = Elem<T>::to_f2(b[j]);
        if (weight_after_cast) {
          const float2 h = Elem<T>::to_f2(Elem<T>::from_f2(f.x * inv, f.y * inv));
          o2[j] = Elem<T>::from_f2(h.x * g.x, h.y * g.y);
        } else {
          o2[j] = Elem<T>::from_f2(g.x * (f.x * inv), g.y * (f.y * inv));
        }
      }
      op[c] = o;
    }
  }
}

// Generic path: any n, any alignment, any dtype; re-reads the row for the second pass.
template <typename T>
__global__ void __launch_bounds__(256) rms_norm_generic_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                                               const T* __restrict__ res, T* __restrict__ out,
                                                               T* __restrict__ out_res, int n, int64_t xs,
                                                               int64_t rs, int64_t os, float eps,
                                                               int weight_after_cast) {
  __shared__ float red[8];
  const int64_t row = blockIdx.x;
  const T* xr = x + row * xs;
  const T* rr = res ? res + row * rs : nullptr;
  T* orr = out_res ? out_res + row * rs : nullptr;
  T* outr = out + row * os;
  float ss = 0.f;
  for (int c = threadIdx.x; c < n; c += 256) {
    T v = xr[c];
    if (rr) {
      v = Elem<T>::from_f(Elem<T>::to_f(v) + Elem<T>::to_f(rr[c]));
      if (orr) orr[c] = v;
      else outr[c] = v;   // parked for the second pass when the caller does not want the sum back
    }
    const float f = Elem<T>::to_f(v);
    ss += f * f;
  }
  const float inv = rsqrtf(block_sum_256(ss, red) * (1.0f / n) + eps);
  for (int c = threadIdx.x; c < n; c += 256) {
    const T v = rr ? (orr ? orr[c] : outr[c]) : xr[c];
    const float f = Elem<T>::to_f(v), g = Elem<T>::to_f(w[c]);
    outr[c] = weight_after_cast ? Elem<T>::from_f(Elem<T>::to_f(Elem<T>::from_f(f * inv)) * g)
                                : Elem<T>::from_f(g * (f * inv));
  }
}

template <typename T>
static int launch_rms(const void* x, const void* w, const void* res, void* out, void* out_res, int64_t rows, int n,
                      int64_t xs, int64_t rs, int64_t os, float eps, int wac, cudaStream_t s) {
  const bool aligned = sizeof(T) == 2 && n % 8 == 0 && xs % 8 == 0 && os % 8 == 0 && (!res || rs % 8 == 0) &&
                       ((((uintptr_t)x | (uintptr_t)w | (uintptr_t)out | (uintptr_t)res | (uintptr_t)out_res) & 15) == 0);
  const T* xp = (const T*)x;
  const T* wp = (const T*)w;
  const T* rp = (const T*)res;
  T* op = (T*)out;
  T* orp = (T*)out_res;
  const unsigned grid = (unsigned)rows;
  if constexpr (sizeof(T) == 2) {
    if (aligned && n <= 16384) {
      const int nvec = n / 8;
      if (nvec <= 256) rms_norm_vec_kernel<T, 1><<<grid, 256, 0, s>>>(xp, wp, rp, op, orp, n, xs, rs, os, eps, wac);
      else if (nvec <= 512) rms_norm_vec_kernel<T, 2><<<grid, 256, 0, s>>>(xp, wp, rp, op, orp, n, xs, rs, os, eps, wac);
      else if (nvec <= 1024) rms_norm_vec_kernel<T, 4><<<grid, 256, 0, s>>>(xp, wp, rp, op, orp, n, xs, rs, os, eps, wac);
      else rms_norm_vec_kernel<T, 8><<<grid, 256, 0, s>>>(xp, wp, rp, op, orp, n, xs, rs, os, eps, wac);
      DLB_CUDA_LAUNCH_CHECK();
      return DLB_OK;
    }
  }
  rms_norm_generic_kernel<T><<<grid, 256, 0, s>>>(xp, wp, rp, op, orp, n, xs, rs, os, eps, wac);
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

// ----------------------------------------------------------------------------
// rotary position embedding (rotate-half convention)
// ----------------------------------------------------------------------------
struct RotaryParams {
  const void *q, *k, *cos, *sin;
  void *qo, *ko;
  int64_t q_st, q_sh, k_st, k_sh, qo_st, qo_sh, ko_st, ko_sh;
  int64_t tokens;
  int hq, hk, dim;
};

// Vector path: 16-bit types, half a head a multiple of 8 elements, 16-byte aligned rows.  One thread
// rotates 8 lower-half and the matching 8 upper-half elements (two 128-bit loads, two stores).
template <typename T> __global__ void __launch_bounds__(256) rotary_vec_kernel(const RotaryParams p) {
  constexpr int TOKENS_PER_CTA = 4;              // enough work per CTA to amortise its launch
  const int half = p.dim >> 1;
  const int hv = half >> 3;                      // vectors per half head
  const int per_token = (p.hq + p.hk) * hv;
  const int64_t t0 = (int64_t)blockIdx.x * TOKENS_PER_CTA;
  const int ntok = (int)min((int64_t)TOKENS_PER_CTA, p.tokens - t0);
  for (int idx = threadIdx.x; idx < ntok * per_token; idx += blockDim.x) {
    const int tl = idx / per_token;
    const int rem = idx - tl * per_token;
    const int64_t t = t0 + tl;
    const int h = rem / hv;
    const int i = rem - h * hv;
    const uint4* cs = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.cos) + t * p.dim);
    const uint4* sn = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.sin) + t * p.dim);
    const T* src;
    T* dst;
    if (h < p.hq) {
      src = reinterpret_cast<const T*>(p.q) + t * p.q_st + (int64_t)h * p.q_sh;
      dst = reinterpret_cast<T*>(p.qo) + t * p.qo_st + (int64_t)h * p.qo_sh;
    } else {
      src = reinterpret_cast<const T*>(p.k) + t * p.k_st + (int64_t)(h - p.hq) * p.k_sh;
      dst = reinterpret_cast<T*>(p.ko) + t * p.ko_st + (int64_t)(h - p.hq) * p.ko_sh;
    }
    const uint4 lo = *(reinterpret_cast<const uint4*>(src) + i);
    const uint4 hi = *(reinterpret_cast<const uint4*>(src + half) + i);
    const uint4 cl = __ldg(cs + i), ch = __ldg(cs + hv + i), sl = __ldg(sn + i), sh = __ldg(sn + hv + i);
    uint4 olo, ohi;
    rot_vec8<T>(lo, hi, cl, ch, sl, sh, olo, ohi);
    *(reinterpret_cast<uint4*>(dst) + i) = olo;
    *(reinterpret_cast<uint4*>(dst + half) + i) = ohi;
  }
}

// One CTA per token; threads sweep (head, element of the lower half).
template <typename T> __global__ void __launch_bounds__(256) rotary_kernel(const RotaryParams p) {
  const int64_t t = blockIdx.x;
  const int half = p.dim >> 1;
  const T* cs = reinterpret_cast<const T*>(p.cos) + t * p.dim;
  const T* sn = reinterpret_cast<const T*>(p.sin) + t * p.dim;
  const int total = (p.hq + p.hk) * half;
  for (int idx = threadIdx.x; idx < total; idx += blockDim.x) {
    const int h = idx / half;
    const int i = idx - h * half;
    const T *src;
    T* dst;
    if (h < p.hq) {
      src = reinterpret_cast<const T*>(p.q) + t * p.q_st + (int64_t)h * p.q_sh;
      dst = reinterpret_cast<T*>(p.qo) + t * p.qo_st + (int64_t)h * p.qo_sh;
    } else {
      src = reinterpret_cast<const T*>(p.k) + t * p.k_st + (int64_t)(h - p.hq) * p.k_sh;
      dst = reinterpret_cast<T*>(p.ko) + t * p.ko_st + (int64_t)(h - p.hq) * p.ko_sh;
    }
    const T lo = src[i], hi = src[half + i];
    dst[i] = rot_lo<T>(lo, hi, cs[i], sn[i]);
    dst[half + i] = rot_hi<T>(lo, hi, cs[half + i], sn[half + i]);
  }
}

// ----------------------------------------------------------------------------
// fill_kv_cache
// ----------------------------------------------------------------------------
struct FillParams {
  const void *ks, *vs;
  void *kc, *vc;
  const void *q_start, *q_len, *kv_len, *table;
  int64_t ks_st, ks_sh, vs_st, vs_sh;           // state strides (token, head), elements
  int64_t kc_sp, kc_ss, kc_sh, vc_sp, vc_ss, vc_sh;   // cache strides (page, slot, head)
  int64_t table_stride;
  int page, heads, dim_k, dim_v, max_pages, num_pages;
  int idx64_start, idx64_len, idx64_kv, idx64_table;
  int elem_size;
  const void *k_cos, *k_sin;     // optional [total tokens, dim_k] rows in the states' dtype: K is rotated on its way in
};

__device__ __forceinline__ int64_t load_idx(const void* p, int64_t i, int is64) {
  return is64 ? reinterpret_cast<const int64_t*>(p)[i] : (int64_t)reinterpret_cast<const int32_t*>(p)[i];
}

// grid (sequence, page index among the pages this step touches); byte-wise copy in 16-byte or 2/4-byte units
template <int UNIT>
__global__ void __launch_bounds__(256) fill_kv_cache_kernel(const FillParams p) {
  const int b = blockIdx.x;
  const int blk = blockIdx.y;
  const int64_t q_start = load_idx(p.q_start, b, p.idx64_start);
  const int q_len = (int)load_idx(p.q_len, b, p.idx64_len);
  const int kv_len = (int)load_idx(p.kv_len, b, p.idx64_kv);
  const int history = kv_len - q_len;
  if (q_len <= 0 || history < 0) return;
  const int first_slot0 = history % p.page;
  const int page_idx = history / p.page + blk;
  if (page_idx >= p.max_pages) return;
  const int slot_lo = blk == 0 ? first_slot0 : 0;
  const int slot_hi = min(p.page, q_len + first_slot0 - blk * p.page);
  if (slot_lo >= slot_hi) return;
  const int64_t page = load_idx(p.table, (int64_t)b * p.table_stride + page_idx, p.idx64_table);
  if (page < 0 || page >= p.num_pages) return;
  const int64_t tok0 = q_start + max(blk * p.page - first_slot0, 0);   // first new token landing in this page
  const int es = p.elem_size;
  const int k_units = p.dim_k * es / UNIT, v_units = p.dim_v * es / UNIT;
  const int per_tok = p.heads * (k_units + v_units);
  const int total = (slot_hi - slot_lo) * per_tok;
  using U = typename std::conditional<UNIT == 16, uint4, typename std::conditional<UNIT == 4, uint32_t, uint16_t>::type>::type;
  // blockIdx.z splits a page; four independent copies in flight per thread
  auto locate = [&](int idx, const U*& src, U*& dst) {
    const int s = idx / per_tok;
    int r = idx - s * per_tok;
    const int slot = slot_lo + s;
    const int64_t tok = tok0 + s;
    if (r < p.heads * k_units) {
      const int h = r / k_units, u = r - h * k_units;
      src = reinterpret_cast<const U*>(reinterpret_cast<const uint8_t*>(p.ks) + (tok * p.ks_st + h * p.ks_sh) * es) + u;
      dst = reinterpret_cast<U*>(reinterpret_cast<uint8_t*>(p.kc) + (page * p.kc_sp + slot * p.kc_ss + h * p.kc_sh) * es) + u;
    } else {
      r -= p.heads * k_units;
      const int h = r / v_units, u = r - h * v_units;
      src = reinterpret_cast<const U*>(reinterpret_cast<const uint8_t*>(p.vs) + (tok * p.vs_st + h * p.vs_sh) * es) + u;
      dst = reinterpret_cast<U*>(reinterpret_cast<uint8_t*>(p.vc) + (page * p.vc_sp + slot * p.vc_ss + h * p.vc_sh) * es) + u;
    }
  };
  const int stride = blockDim.x * gridDim.z;
  if (stride % per_tok == 0) {
    // A thread keeps its (head, unit) column and walks the slots, four copies in flight: the index
    // arithmetic (two divisions per unit in the general walk below) is done once per thread.
    const int idx0 = threadIdx.x + blockIdx.z * blockDim.x;
    const int s0 = idx0 / per_tok, ds = stride / per_tok;
    int r = idx0 - s0 * per_tok;
    const uint8_t* sbase;
    uint8_t* dbase;
    int64_t s_tok, d_slot;     // bytes per token of the states / per slot of the cache
    if (r < p.heads * k_units) {
      const int h = r / k_units, u = r - h * k_units;
      sbase = reinterpret_cast<const uint8_t*>(p.ks) + ((int64_t)h * p.ks_sh) * es + (int64_t)u * UNIT;
      dbase = reinterpret_cast<uint8_t*>(p.kc) + (page * p.kc_sp + (int64_t)h * p.kc_sh) * es + (int64_t)u * UNIT;
      s_tok = p.ks_st * es;
      d_slot = p.kc_ss * es;
    } else {
      r -= p.heads * k_units;
      const int h = r / v_units, u = r - h * v_units;
      sbase = reinterpret_cast<const uint8_t*>(p.vs) + ((int64_t)h * p.vs_sh) * es + (int64_t)u * UNIT;
      dbase = reinterpret_cast<uint8_t*>(p.vc) + (page * p.vc_sp + (int64_t)h * p.vc_sh) * es + (int64_t)u * UNIT;
      s_tok = p.vs_st * es;
      d_slot = p.vc_ss * es;
    }
    const int nslots = slot_hi - slot_lo;
    for (int sidx = s0; sidx < nslots; sidx += 4 * ds) {
      U val[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (sidx + j * ds < nslots) val[j] = *reinterpret_cast<const U*>(sbase + (tok0 + sidx + j * ds) * s_tok);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (sidx + j * ds < nslots) *reinterpret_cast<U*>(dbase + (int64_t)(slot_lo + sidx + j * ds) * d_slot) = val[j];
    }
    return;
  }
  for (int idx = threadIdx.x + blockIdx.z * blockDim.x; idx < total; idx += 4 * stride) {
    const U* src[4];
    U* dst[4];
    U val[4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (idx + j * stride < total) locate(idx + j * stride, src[j], dst[j]);
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (idx + j * stride < total) val[j] = *src[j];
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if (idx + j * stride < total) *dst[j] = val[j];
  }
}

// The same walk with the rotary embedding of K applied on the way (rotate-half convention, arithmetic in the
// 16-bit type, bit-identical to apply_rotary followed by a plain fill): one work item is a (lower, upper) pair
// of 16-byte chunks of a K row, or one 16-byte chunk of a V row.  The cache then holds rotated keys, so the
// attention kernels need no pass over K before they read it.
template <typename T>
__global__ void __launch_bounds__(512, 3) fill_kv_cache_rot_kernel(const FillParams p) {
  const int b = blockIdx.x;
  const int blk = blockIdx.y;
  const int64_t q_start = load_idx(p.q_start, b, p.idx64_start);
  const int q_len = (int)load_idx(p.q_len, b, p.idx64_len);
  const int kv_len = (int)load_idx(p.kv_len, b, p.idx64_kv);
  const int history = kv_len - q_len;
  if (q_len <= 0 || history < 0) return;
  const int first_slot0 = history % p.page;
  const int page_idx = history / p.page + blk;
  if (page_idx >= p.max_pages) return;
  const int slot_lo = blk == 0 ? first_slot0 : 0;
  const int slot_hi = min(p.page, q_len + first_slot0 - blk * p.page);
  if (slot_lo >= slot_hi) return;
  const int64_t page = load_idx(p.table, (int64_t)b * p.table_stride + page_idx, p.idx64_table);
  if (page < 0 || page >= p.num_pages) return;
  const int64_t tok0 = q_start + max(blk * p.page - first_slot0, 0);
  const int half = p.dim_k >> 1, hv = half >> 3, v_units = p.dim_v >> 3;
  const int per_tok = p.heads * (hv + v_units);
  // The block size is a multiple of per_tok (the launcher sees to it), so a thread keeps its item of the
  // token row (a K chunk pair of one head, or a V chunk) and walks the slots: no division inside the loop.
  const int idx0 = threadIdx.x + blockIdx.z * blockDim.x;
  const int s0 = idx0 / per_tok, ds = (blockDim.x * gridDim.z) / per_tok;
  int r = idx0 - s0 * per_tok;
  const int nslots = slot_hi - slot_lo;
  if (r < p.heads * hv) {
    const int h = r / hv, i = r - h * hv;
    const T* sbase = reinterpret_cast<const T*>(p.ks) + (int64_t)h * p.ks_sh;
    T* dbase = reinterpret_cast<T*>(p.kc) + page * p.kc_sp + (int64_t)h * p.kc_sh;
#pragma unroll 1
    for (int sidx = s0; sidx < nslots; sidx += ds) {
      const int64_t tok = tok0 + sidx;
      const T* src = sbase + tok * p.ks_st;
      T* dst = dbase + (int64_t)(slot_lo + sidx) * p.kc_ss;
      const T* cs = reinterpret_cast<const T*>(p.k_cos) + tok * p.dim_k;
      const T* sn = reinterpret_cast<const T*>(p.k_sin) + tok * p.dim_k;
      const uint4 lo = *(reinterpret_cast<const uint4*>(src) + i);
      const uint4 hi = *(reinterpret_cast<const uint4*>(src + half) + i);
      const uint4 cl = __ldg(reinterpret_cast<const uint4*>(cs) + i), ch = __ldg(reinterpret_cast<const uint4*>(cs + half) + i);
      const uint4 sl = __ldg(reinterpret_cast<const uint4*>(sn) + i), sh = __ldg(reinterpret_cast<const uint4*>(sn + half) + i);
      uint4 olo, ohi;
      rot_vec8<T>(lo, hi, cl, ch, sl, sh, olo, ohi);
      *(reinterpret_cast<uint4*>(dst) + i) = olo;
      *(reinterpret_cast<uint4*>(dst + half) + i) = ohi;
    }
  } else {
    r -= p.heads * hv;
    const int h = r / v_units, u = r - h * v_units;
    const T* sbase = reinterpret_cast<const T*>(p.vs) + (int64_t)h * p.vs_sh;
    T* dbase = reinterpret_cast<T*>(p.vc) + page * p.vc_sp + (int64_t)h * p.vc_sh;
    for (int sidx = s0; sidx < nslots; sidx += 4 * ds) {
      uint4 val[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (sidx + j * ds < nslots) val[j] = *(reinterpret_cast<const uint4*>(sbase + (tok0 + sidx + j * ds) * p.vs_st) + u);
#pragma unroll
      for (int j = 0; j < 4; ++j)
        if (sidx + j * ds < nslots) *(reinterpret_cast<uint4*>(dbase + (int64_t)(slot_lo + sidx + j * ds) * p.vc_ss) + u) = val[j];
    }
  }
}

}  // namespace dlb

extern "C" int dlb_rms_norm(const void* x, const void* weight, const void* residual, void* out, void* out_residual,
                            int64_t rows, int64_t n, int64_t x_row_stride, int64_t residual_row_stride,
                            int64_t out_row_stride, float eps, int weight_after_cast, int dtype, void* stream) {
  DLB_NVTX("dlb_rms_norm");
  using namespace dlb;
  DLB_CHECK_ARG(rows >= 0 && n >= 1 && n < (1LL << 30), DLB_ERR_BAD_ARG, "rms_norm: bad sizes");
  if (rows == 0) return DLB_OK;
  DLB_CHECK_ARG(rows < (1LL << 31), DLB_ERR_TOO_LARGE, "rms_norm: too many rows");
  DLB_CHECK_ARG(x && weight && out, DLB_ERR_BAD_ARG, "rms_norm: null pointer");
  DLB_CHECK_ARG(out_residual == nullptr || residual != nullptr, DLB_ERR_BAD_ARG,
                "rms_norm: out_residual needs a residual");
  cudaStream_t s = (cudaStream_t)stream;
  switch (dtype) {
    case DLB_DTYPE_BF16:
      return launch_rms<__nv_bfloat16>(x, weight, residual, out, out_residual, rows, (int)n, x_row_stride,
                                       residual_row_stride, out_row_stride, eps, weight_after_cast, s);
    case DLB_DTYPE_F16:
      return launch_rms<__half>(x, weight, residual, out, out_residual, rows, (int)n, x_row_stride,
                                residual_row_stride, out_row_stride, eps, weight_after_cast, s);
    case DLB_DTYPE_F32:
      return launch_rms<float>(x, weight, residual, out, out_residual, rows, (int)n, x_row_stride,
                               residual_row_stride, out_row_stride, eps, weight_after_cast, s);
    default:
      set_last_error("rms_norm: unsupported dtype %d", dtype);
      return DLB_ERR_UNSUPPORTED;
  }
}

extern "C" int dlb_apply_rotary(const void* q, const void* k, const void* cos, const void* sin, void* q_out,
                                void* k_out, int64_t tokens, int hq, int hk, int dim, int64_t q_stride_t,
                                int64_t q_stride_h, int64_t k_stride_t, int64_t k_stride_h, int64_t qo_stride_t,
                                int64_t qo_stride_h, int64_t ko_stride_t, int64_t ko_stride_h, int dtype,
                                void* stream) {
  DLB_NVTX("dlb_apply_rotary");
  using namespace dlb;
  DLB_CHECK_ARG(tokens >= 0 && hq >= 0 && hk >= 0 && dim >= 2 && dim % 2 == 0, DLB_ERR_BAD_ARG, "rotary: bad sizes");
  if (tokens == 0 || hq + hk == 0) return DLB_OK;
  DLB_CHECK_ARG(tokens < (1LL << 31), DLB_ERR_TOO_LARGE, "rotary: too many tokens");
  DLB_CHECK_ARG(cos && sin && (hq == 0 || (q && q_out)) && (hk == 0 || (k && k_out)), DLB_ERR_BAD_ARG,
                "rotary: null pointer");
  RotaryParams p{q, k, cos, sin, q_out, k_out, q_stride_t, q_stride_h, k_stride_t, k_stride_h,
                 qo_stride_t, qo_stride_h, ko_stride_t, ko_stride_h, tokens, hq, hk, dim};
  cudaStream_t s = (cudaStream_t)stream;
  const bool vec = dtype != DLB_DTYPE_F32 && (dim / 2) % 8 == 0 &&
                   ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)q_out | (uintptr_t)k_out | (uintptr_t)cos |
                      (uintptr_t)sin) & 15) == 0) &&
                   q_stride_t % 8 == 0 && q_stride_h % 8 == 0 && k_stride_t % 8 == 0 && k_stride_h % 8 == 0 &&
                   qo_stride_t % 8 == 0 && qo_stride_h % 8 == 0 && ko_stride_t % 8 == 0 && ko_stride_h % 8 == 0;
  if (vec) {
    const unsigned blocks = (unsigned)((tokens + 3) / 4);     // TOKENS_PER_CTA = 4
    if (dtype == DLB_DTYPE_BF16) rotary_vec_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(p);
    else rotary_vec_kernel<__half><<<blocks, 256, 0, s>>>(p);
    DLB_CUDA_LAUNCH_CHECK();
    return DLB_OK;
  }
  const int work = (hq + hk) * (dim / 2);
  const int threads = work >= 256 ? 256 : ((work + 31) / 32) * 32;
  switch (dtype) {
    case DLB_DTYPE_BF16: rotary_kernel<__nv_bfloat16><<<(unsigned)tokens, threads, 0, s>>>(p); break;
    case DLB_DTYPE_F16: rotary_kernel<__half><<<(unsigned)tokens, threads, 0, s>>>(p); break;
    case DLB_DTYPE_F32: rotary_kernel<float><<<(unsigned)tokens, threads, 0, s>>>(p); break;
    default:
      set_last_error("rotary: unsupported dtype %d", dtype);
      return DLB_ERR_UNSUPPORTED;
  }
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

extern "C" int dlb_fill_kv_cache(const void* k_states, const void* v_states, void* k_caches, void* v_caches,
                                 const void* q_start_loc, const void* q_seq_length, const void* kv_seq_length,
                                 const void* block_offsets, int64_t batch, int64_t max_q_seq_length,
                                 int64_t page_size, int64_t heads, int64_t dim_k, int64_t dim_v, int64_t num_pages,
                                 int64_t max_pages, int64_t ks_stride_t, int64_t ks_stride_h, int64_t vs_stride_t,
                                 int64_t vs_stride_h, int64_t kc_stride_page, int64_t kc_stride_slot,
                                 int64_t kc_stride_head, int64_t vc_stride_page, int64_t vc_stride_slot,
                                 int64_t vc_stride_head, int64_t table_stride, int start_is_int64, int qlen_is_int64,
                                 int kvlen_is_int64, int table_is_int64, int elem_size, const void* k_cos,
                                 const void* k_sin, int dtype, void* stream) {
  DLB_NVTX("dlb_fill_kv_cache");
  using namespace dlb;
  DLB_CHECK_ARG(batch >= 0 && max_q_seq_length >= 0 && page_size >= 1 && heads >= 1 && dim_k >= 1 && dim_v >= 0,
                DLB_ERR_BAD_ARG, "fill_kv_cache: bad sizes");
  DLB_CHECK_ARG(elem_size == 1 || elem_size == 2 || elem_size == 4, DLB_ERR_UNSUPPORTED,
                "fill_kv_cache: element size %d", elem_size);
  if (batch == 0 || max_q_seq_length == 0) return DLB_OK;
  DLB_CHECK_ARG(k_states && v_states && k_caches && v_caches && q_start_loc && q_seq_length && kv_seq_length &&
                    block_offsets,
                DLB_ERR_BAD_ARG, "fill_kv_cache: null pointer");
  const int64_t blocks = (max_q_seq_length + page_size - 1) / page_size + 1;
  DLB_CHECK_ARG(batch < (1LL << 31) && blocks <= 65535, DLB_ERR_TOO_LARGE, "fill_kv_cache: grid too large");
  FillParams p;
  p.ks = k_states; p.vs = v_states; p.kc = k_caches; p.vc = v_caches;
  p.q_start = q_start_loc; p.q_len = q_seq_length; p.kv_len = kv_seq_length; p.table = block_offsets;
  p.ks_st = ks_stride_t; p.ks_sh = ks_stride_h; p.vs_st = vs_stride_t; p.vs_sh = vs_stride_h;
  p.kc_sp = kc_stride_page; p.kc_ss = kc_stride_slot; p.kc_sh = kc_stride_head;
  p.vc_sp = vc_stride_page; p.vc_ss = vc_stride_slot; p.vc_sh = vc_stride_head;
  p.table_stride = table_stride;
  p.page = (int)page_size; p.heads = (int)heads; p.dim_k = (int)dim_k; p.dim_v = (int)dim_v;
  p.max_pages = (int)max_pages; p.num_pages = (int)num_pages;
  p.idx64_start = start_is_int64; p.idx64_len = qlen_is_int64; p.idx64_kv = kvlen_is_int64;
  p.idx64_table = table_is_int64;
  p.elem_size = elem_size;
  p.k_cos = k_cos;
  p.k_sin = k_sin;
  DLB_CHECK_ARG((k_cos == nullptr) == (k_sin == nullptr), DLB_ERR_BAD_ARG, "fill_kv_cache: cos and sin go together");
  // widest copy unit that every row start and row length allows
  auto mult = [&](int64_t v, int unit) { return (v * elem_size) % unit == 0; };
  const uintptr_t ptrs = (uintptr_t)k_states | (uintptr_t)v_states | (uintptr_t)k_caches | (uintptr_t)v_caches;
  bool ok16 = (ptrs & 15) == 0;
  for (int64_t v : {dim_k, dim_v, ks_stride_t, ks_stride_h, vs_stride_t, vs_stride_h, kc_stride_page, kc_stride_slot,
                    kc_stride_head, vc_stride_page, vc_stride_slot, vc_stride_head})
    ok16 = ok16 && mult(v, 16);
  // a page's slots are cut into 4 pieces (plain copy) or 8 (rotating form); measured on 4 x 8192 tokens:
  // plain 4 / 8 / 16 pieces -> 47.7 / 49 / 53 us, rotating 1 / 2 / 4 / 8 / 16 -> 58 / 57 / 56 / 53 / 58 us
  dim3 grid((unsigned)batch, (unsigned)blocks, k_cos != nullptr ? 8 : 4);
  cudaStream_t s = (cudaStream_t)stream;
  if (k_cos != nullptr) {
    DLB_CHECK_ARG(ok16 && elem_size == 2 && dim_k % 16 == 0 && (dtype == DLB_DTYPE_BF16 || dtype == DLB_DTYPE_F16) &&
                      (((uintptr_t)k_cos | (uintptr_t)k_sin) & 15) == 0,
                  DLB_ERR_UNSUPPORTED,
                  "fill_kv_cache: rotating K needs fp16/bf16, a head size that is a multiple of 16 and 16-byte aligned rows");
    const int per_tok = (int)(heads * (dim_k / 16 + dim_v / 8));
    DLB_CHECK_ARG(per_tok <= 512, DLB_ERR_UNSUPPORTED, "fill_kv_cache: heads x head size too large for the rotating form");
    const int threads = (512 / per_tok) * per_tok;      // a multiple of per_tok: every thread keeps its item
    if (dtype == DLB_DTYPE_BF16) fill_kv_cache_rot_kernel<__nv_bfloat16><<<grid, threads, 0, s>>>(p);
    else fill_kv_cache_rot_kernel<__half><<<grid, threads, 0, s>>>(p);
    DLB_CUDA_LAUNCH_CHECK();
    return DLB_OK;
  }
  if (ok16) fill_kv_cache_kernel<16><<<grid, 256, 0, s>>>(p);
  else if (elem_size == 4) fill_kv_cache_kernel<4><<<grid, 256, 0, s>>>(p);
  else if (elem_size == 2) fill_kv_cache_kernel<2><<<grid, 256, 0, s>>>(p);
  else {
    set_last_error("fill_kv_cache: 1-byte elements need 16-byte aligned rows");
    return DLB_ERR_ALIGNMENT;
  }
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}
