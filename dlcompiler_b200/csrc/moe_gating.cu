// MoE router: grouped top-k gating (DeepSeek-V3 style) and plain softmax top-k.
//
// One warp per token.  Lane l owns the VPL consecutive experts
// [l*VPL, (l+1)*VPL), loaded as 128-bit vectors; every reduction (softmax
// max/sum, per-group top-2 sums, group ranking, k rounds of arg-max) is a
// warp-shuffle tree or a hardware warp reduction; shared memory only holds
// per-warp lists (no atomics), so the result is deterministic.
//
// Algorithm (scoring = sigmoid, grouped):
//   s[e]   = sigmoid(logits[e])                       (weights come from s)
//   c[e]   = s[e] + bias[e]                            (selection score)
//   g[j]   = sum of the two largest c in group j
//   keep the topk_group groups with the largest g (ties: lower group index)
//   pick the top_k experts with the largest c among kept groups
//     (ties: lower expert index), output in descending order of c
//   w[i]   = s[id_i]; if renormalize: w /= sum(w) (+eps); w *= scale
// With scoring = softmax and n_group = topk_group = 1 this is the
// softmax -> top-k router the fused_moe tests build with torch
// (python/dlBLAS/tests/kernels/test_fused_moe.py:207-218).
#include <math_constants.h>

#include "common.cuh"

namespace dlb {

#define DLB_SCORE_SIGMOID 0
#define DLB_SCORE_SOFTMAX 1

struct GatingParams {
  const float* logits;   // [T, E] row stride = ld
  const float* bias;     // [E] or null
  int32_t* ids;          // [T, K]
  float* weights;        // [T, K]
  float* probs;          // optional [T, E] output of the un-biased scores (softmax probabilities / sigmoid)
  int64_t tokens;
  int64_t ld;
  int experts;
  int n_group;
  int topk_group;
  int top_k;
  int scoring;
  int renormalize;
  float scale;
  int lanes_per_group = 1;        // filled by launch_gating
  int lanes_per_group_log2 = 0;
};

// sigmoid evaluated by a FIXED sequence of correctly-rounded fp32 operations (fused
// multiply-add, add, sub, integer add/sub on bit patterns; no division, no
// approximate transcendental), so that the CPU checker, which performs the same sequence
// with an exact fp32 FMA, gets bit-identical scores and therefore bit-identical expert ids
// even for near-ties:
//   xc = clamp(x, -87, 86);  z = fma(xc, -log2e, M);  n = z - M          (M = 1.5 * 2^23)
//   r  = fma(xc, -log2e_lo, fma(xc, -log2e_hi, -n))                        (|r| <= 0.5)
//   p  = 2^r by a degree-5 Horner scheme of FMAs;  e = p * 2^n (n added to p's exponent bits)
//   d  = 1 + e;  y = bits^-1(0x7EF311C7 - bits(d));  three Newton steps y = fma(y, fma(-d, y, 1), y)
//   sigmoid = y   (no division, no branch)
__device__ __forceinline__ float sigmoid_spec(float x) {
  constexpr float kMagic = 12582912.0f;
  constexpr float kNegLog2eHi = -1.44269502162933349609e+00f;
  constexpr float kNegLog2eLo = -1.92596303350001107901e-08f;
  const float xc = fminf(fmaxf(x, -87.0f), 86.0f);
  const float z = __fmaf_rn(xc, kNegLog2eHi, kMagic);
  const float n = __fsub_rn(z, kMagic);
  float r = __fmaf_rn(xc, kNegLog2eHi, -n);
  r = __fmaf_rn(xc, kNegLog2eLo, r);
  float p = 1.32874317932873964310e-03f;
  p = __fmaf_rn(p, r, 9.67150740325450897217e-03f);
  p = __fmaf_rn(p, r, 5.55065572261810302734e-02f);
  p = __fmaf_rn(p, r, 2.40222424268722534180e-01f);
  p = __fmaf_rn(p, r, 6.93147063255310058594e-01f);
  p = __fmaf_rn(p, r, 1.0f);
  const float e = __int_as_float(__float_as_int(p) + (__float_as_int(z) << 23));
  const float d = __fadd_rn(1.0f, e);
  float y = __int_as_float(0x7EF311C7 - __float_as_int(d));   // 5 % first guess of 1/d
#pragma unroll
  for (int it = 0; it < 3; ++it) y = __fmaf_rn(y, __fmaf_rn(-d, y, 1.0f), y);   // 5e-2 -> 2.5e-3 -> 6e-6 -> rounding
  return y;
}

// The same sequence on two scores at once with the packed fp32 instructions of sm_100 (fma.rn.f32x2,
// add.rn.f32x2): every lane of a packed operation rounds exactly like its scalar form, so the scores are
// bit-identical to sigmoid_spec, and the 16 FMAs / adds of the sequence cost half the issue slots.
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
// The packed constants of the sequence, as 64-bit pairs in constant memory: the compiler keeps them in
// uniform registers, where immediates would be rebuilt pair by pair with moves.
enum { SC_HI = 0, SC_LO, SC_MAGIC, SC_NEG1, SC_ONE, SC_P5, SC_P4, SC_P3, SC_P2, SC_P1, SC_COUNT };
__constant__ float2 g_sig_pairs[SC_COUNT] = {
    {-1.44269502162933349609e+00f, -1.44269502162933349609e+00f}, {-1.92596303350001107901e-08f, -1.92596303350001107901e-08f},
    {12582912.0f, 12582912.0f}, {-1.0f, -1.0f}, {1.0f, 1.0f},
    {1.32874317932873964310e-03f, 1.32874317932873964310e-03f}, {9.67150740325450897217e-03f, 9.67150740325450897217e-03f},
    {5.55065572261810302734e-02f, 5.55065572261810302734e-02f}, {2.40222424268722534180e-01f, 2.40222424268722534180e-01f},
    {6.93147063255310058594e-01f, 6.93147063255310058594e-01f}};
__device__ __forceinline__ uint64_t sig_pair(int i) { return *reinterpret_cast<const uint64_t*>(&g_sig_pairs[i]); }
// Packed sigmoid_spec of two logits; the result stays packed (lo = sigmoid(x0), hi = sigmoid(x1)).
__device__ __forceinline__ uint64_t sigmoid_spec2(float x0, float x1) {
  const float c0 = fminf(fmaxf(x0, -87.0f), 86.0f), c1 = fminf(fmaxf(x1, -87.0f), 86.0f);
  const uint64_t xc = f2_pack(c0, c1);
  const uint64_t hi2 = sig_pair(SC_HI), magic2 = sig_pair(SC_MAGIC), neg1 = sig_pair(SC_NEG1), one = sig_pair(SC_ONE);
  const uint64_t z = f2_fma(xc, hi2, magic2);
  const uint64_t negn = f2_fma(z, neg1, magic2);                                 // M - z = -n, exact
  uint64_t r = f2_fma(xc, hi2, negn);
  r = f2_fma(xc, sig_pair(SC_LO), r);
  uint64_t p = sig_pair(SC_P5);
  p = f2_fma(p, r, sig_pair(SC_P4));
  p = f2_fma(p, r, sig_pair(SC_P3));
  p = f2_fma(p, r, sig_pair(SC_P2));
  p = f2_fma(p, r, sig_pair(SC_P1));
  p = f2_fma(p, r, one);
  float p0, p1, z0, z1;
  f2_unpack(p, p0, p1);
  f2_unpack(z, z0, z1);
  // e = p * 2^n: n sits in the low bits of z; one integer multiply-add moves it into p's exponent field
  const uint32_t e0 = __float_as_uint(z0) * 0x00800000u + __float_as_uint(p0);
  const uint32_t e1 = __float_as_uint(z1) * 0x00800000u + __float_as_uint(p1);
  // -d = -(1 + e) rounds exactly like d (round-to-nearest is symmetric); bits(d) = bits(-d) - 2^31, so the
  // first guess 0x7EF311C7 - bits(d) is 0xFEF311C7 - bits(-d) and d itself is never needed
  const uint64_t nd = f2_fma(f2_pack(__uint_as_float(e0), __uint_as_float(e1)), neg1, neg1);
  float nd0, nd1;
  f2_unpack(nd, nd0, nd1);
  uint64_t y = f2_pack(__uint_as_float(0xFEF311C7u - __float_as_uint(nd0)),
                       __uint_as_float(0xFEF311C7u - __float_as_uint(nd1)));
#pragma unroll
  for (int it = 0; it < 3; ++it) y = f2_fma(y, f2_fma(nd, y, one), y);
  return y;
}

// Order-preserving map from fp32 to unsigned: a > b  <=>  key(a) > key(b); -inf maps to
// 0x007fffff, which leaves 0 free as "slot retired".
__device__ __forceinline__ uint32_t score_key(float v) {
  const uint32_t b = __float_as_uint(v);
  return b ^ ((uint32_t)((int32_t)b >> 31) | 0x80000000u);     // negative: all bits flip; else only the sign bit
}
constexpr uint32_t KEY_NEG_INF = 0x007fffffu;

// Sorts N keys (unsigned or float) in registers, descending, with Batcher's odd-even merge network
// (19 compare-exchanges for N = 8); every index below is a compile-time constant once unrolled.
template <int N, typename K> __device__ __forceinline__ void sort_desc(K (&k)[N]) {
#pragma unroll
  for (int p = 1; p < N; p <<= 1) {
#pragma unroll
    for (int q = p; q >= 1; q >>= 1) {
#pragma unroll
      for (int j = q % p; j <= N - 1 - q; j += 2 * q) {
#pragma unroll
        for (int i = 0; i < q; ++i) {
          const int lo = i + j, hi = i + j + q;
          if (hi < N && (lo / (2 * p)) == (hi / (2 * p))) {
            const K a = k[lo], b = k[hi];
            k[lo] = max(a, b);
            k[hi] = min(a, b);
          }
        }
      }
    }
  }
}

__device__ __forceinline__ void merge_top2(float& a1, float& a2, float b1, float b2) {
  // (a1 >= a2), (b1 >= b2) -> two largest of the four
  const float hi = fmaxf(a1, b1);
  const float lo = fmaxf(fminf(a1, b1), fmaxf(a2, b2));
  a1 = hi;
  a2 = lo;
}

// Shared-memory shape of the router for VPL experts per lane: a lane's sorted list has VPL entries plus a
// zero terminator, padded so that 128-bit stores stay aligned and (for VPL = 8: 12 words per lane) free of
// bank conflicts; 16 experts per lane run 4 warps per CTA to stay inside the 48 KiB static limit.
template <int VPL> struct GateShape {
  static constexpr int WARPS = VPL >= 16 ? 4 : 8;
  static constexpr int LIST = VPL + (VPL >= 4 ? 4 : 1);
};

// k rounds over the heads of the sorted per-lane lists.  Only the head lives in a register; the rest of a
// lane's list is in shared memory behind it.  One hardware warp reduction (redux.sync) finds the maximum
// head; a ballot picks the lowest lane among equals (lanes hold ascending expert ranges); that lane alone
// records the round's winner as (key, lane, run) in win[k], steps its list pointer and reloads its head
// (the list ends in 0 = retired).  `run` counts how many equal keys of that lane left directly before:
// equal keys inside one lane leave in consecutive rounds and stand for ascending expert indices.
template <bool TRACK_DUP, int TOPK>
__device__ __forceinline__ void topk_rounds(uint32_t head, const uint32_t* __restrict__ my_list, uint2* __restrict__ win,
                                            int top_k_rt, int lane) {
  const int top_k = TOPK > 0 ? TOPK : top_k_rt;
  uint32_t lt;
  asm("mov.u32 %0, %%lanemask_lt;" : "=r"(lt));
  int run = 0;
  uint32_t last = 0;
  uint32_t tag = (uint32_t)lane;     // with `head` the pair that a winner stores: both stay in vector registers
  const uint32_t* next = my_list;    // the lane's list entry behind `head`
#pragma unroll(TOPK > 0 ? TOPK : 4)
  for (int k = 0; k < top_k; ++k) {
    const uint32_t wmax = __reduce_max_sync(0xffffffffu, head);
    const bool mine = head == wmax;
    const uint32_t eq = __ballot_sync(0xffffffffu, mine);
    if (mine && (eq & lt) == 0) {
      if constexpr (TRACK_DUP) {
        run = (head == last) ? run + 1 : 0;
        last = head;
        tag = (uint32_t)lane | ((uint32_t)run << 8);
      }
      win[k] = make_uint2(head, tag);
      ++next;
      head = *next;
    }
  }
}

// One warp per token, VPL experts per lane (lane l holds experts l*VPL ..).  FULL: experts == 32 * VPL
// and 16-byte aligned rows and bias, so no bounds checks and only vector loads.  LG >= 0 fixes the lanes per
// group at 2^LG with all 32 lanes in groups, and TOPK > 0 fixes top_k, so that the shuffle trees, the group
// ranking and the rounds unroll (the DeepSeek-V3 shape: 256 experts, 8 groups, top-8); LG = -1 / TOPK = 0
// read them from the parameters.
constexpr int kGateMinBlocks = 6;   // 40 registers per thread, six CTAs per SM (1 % faster than 48 registers / five)
template <int VPL, bool FULL, int LG = -1, int TOPK = 0>
__global__ void __launch_bounds__(GateShape<VPL>::WARPS * 32, LG >= 0 ? kGateMinBlocks : 1)
grouped_topk_kernel(GatingParams p) {
  constexpr int WARPS = GateShape<VPL>::WARPS, LIST = GateShape<VPL>::LIST;
  const int lane = threadIdx.x & 31;
  const int64_t token = (int64_t)blockIdx.x * WARPS + (threadIdx.x >> 5);
  __shared__ __align__(16) uint32_t sm_key[WARPS][32 * VPL];     // per warp: every expert's selection key, by expert index
  __shared__ __align__(16) float sm_s[WARPS][32 * VPL];          // per warp: every expert's un-biased score
  __shared__ __align__(16) uint32_t sm_list[WARPS][32 * LIST];   // per warp: each lane's keys sorted descending, then 0
  __shared__ __align__(8) uint2 sm_win[WARPS][32];               // per warp: round k's winner (key, lane | run << 8)
  if (token >= p.tokens) return;  // whole warp leaves together

  const int E = p.experts;
  const int e0 = lane * VPL;
  const float* row = p.logits + token * p.ld;
  auto valid = [&](int v) { return FULL || e0 + v < E; };

  float s[VPL];  // un-biased score (sigmoid or softmax probability)
  float c[VPL];  // selection score
  // ---- load ----
  if constexpr (VPL >= 4) {
#pragma unroll
    for (int v = 0; v < VPL; v += 4) {
      if (FULL || e0 + v + 3 < E) {
        const float4 x = __ldg(reinterpret_cast<const float4*>(row + e0 + v));
        s[v] = x.x; s[v + 1] = x.y; s[v + 2] = x.z; s[v + 3] = x.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) s[v + j] = (e0 + v + j < E) ? __ldg(row + e0 + v + j) : -CUDART_INF_F;
      }
    }
  } else {
#pragma unroll
    for (int v = 0; v < VPL; ++v) s[v] = valid(v) ? __ldg(row + e0 + v) : -CUDART_INF_F;
  }

  // ---- scoring ----
  if (LG >= 0 || p.scoring == DLB_SCORE_SIGMOID) {   // the fixed-shape form is only launched for sigmoid scoring
    if constexpr (VPL >= 2) {
#pragma unroll
      for (int v = 0; v < VPL; v += 2) {
        float y0, y1;
        f2_unpack(sigmoid_spec2(s[v], s[v + 1]), y0, y1);
        s[v] = valid(v) ? y0 : -CUDART_INF_F;
        s[v + 1] = valid(v + 1) ? y1 : -CUDART_INF_F;
      }
    } else {
#pragma unroll
      for (int v = 0; v < VPL; ++v) s[v] = valid(v) ? sigmoid_spec(s[v]) : -CUDART_INF_F;
    }
  } else {
    // softmax is monotone in the logit: without a bias the selection runs on the raw logits,
    // which keeps the chosen ids independent of how exp() rounds
    if (p.bias == nullptr) {
#pragma unroll
      for (int v = 0; v < VPL; ++v) c[v] = s[v];
    }
    float m = -CUDART_INF_F;
#pragma unroll
    for (int v = 0; v < VPL; ++v) m = fmaxf(m, s[v]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float sum = 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      s[v] = valid(v) ? expf(s[v] - m) : 0.f;
      sum += s[v];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
    for (int v = 0; v < VPL; ++v) s[v] = valid(v) ? s[v] / sum : -CUDART_INF_F;
  }
  if (p.probs != nullptr) {
#pragma unroll
    for (int v = 0; v < VPL; ++v)
      if (valid(v)) p.probs[token * E + e0 + v] = s[v];
  }
  if (LG >= 0 || p.scoring == DLB_SCORE_SIGMOID || p.bias != nullptr) {
    if (p.bias == nullptr) {
#pragma unroll
      for (int v = 0; v < VPL; ++v) c[v] = s[v];
    } else if constexpr (FULL && VPL >= 4) {
#pragma unroll
      for (int v = 0; v < VPL; v += 4) {
        const float4 bv = __ldg(reinterpret_cast<const float4*>(p.bias + e0 + v));
        f2_unpack(f2_add(f2_pack(s[v], s[v + 1]), f2_pack(bv.x, bv.y)), c[v], c[v + 1]);          // rounds like __fadd_rn
        f2_unpack(f2_add(f2_pack(s[v + 2], s[v + 3]), f2_pack(bv.z, bv.w)), c[v + 2], c[v + 3]);
      }
    } else {
#pragma unroll
      for (int v = 0; v < VPL; ++v) c[v] = valid(v) ? __fadd_rn(s[v], __ldg(p.bias + e0 + v)) : -CUDART_INF_F;
    }
  }

  // ---- keys: the originals go to shared memory for the final index look-up, a sorted copy feeds the rounds.
  // The scores are sorted as floats.  Positive floats order like their bit patterns, so when every selection
  // score of the token is > 0 (sigmoid scores with the usual small bias) the bits serve as integer keys as
  // they are; only a token with a score <= 0 (or -inf fillers of a ragged last lane) pays for the mapping.
  float f[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) f[v] = c[v];
  sort_desc<VPL>(f);
  const bool any_nonpos = __any_sync(0xffffffffu, !(f[VPL - 1] > 0.f));
  uint32_t key[VPL], okey[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    key[v] = __float_as_uint(f[v]);
    okey[v] = __float_as_uint(c[v]);
  }
  if (any_nonpos) {
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      key[v] = score_key(f[v]);
      okey[v] = score_key(c[v]);
    }
  }
  uint32_t* wkeys = sm_key[threadIdx.x >> 5];
  float* wscores = sm_s[threadIdx.x >> 5];
  if constexpr (VPL >= 4) {
#pragma unroll
    for (int v = 0; v < VPL; v += 4) {
      *reinterpret_cast<uint4*>(wkeys + e0 + v) = make_uint4(okey[v], okey[v + 1], okey[v + 2], okey[v + 3]);
      *reinterpret_cast<float4*>(wscores + e0 + v) = make_float4(s[v], s[v + 1], s[v + 2], s[v + 3]);
    }
  } else {
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      wkeys[e0 + v] = okey[v];
      wscores[e0 + v] = s[v];
    }
  }
  uint32_t* my_list = sm_list[threadIdx.x >> 5] + lane * LIST;
  if constexpr (VPL >= 4) {
#pragma unroll
    for (int v = 0; v < VPL; v += 4)
      *reinterpret_cast<uint4*>(my_list + v) = make_uint4(key[v], key[v + 1], key[v + 2], key[v + 3]);
  } else {
#pragma unroll
    for (int v = 0; v < VPL; ++v) my_list[v] = key[v];
  }
  my_list[VPL] = 0u;
  // equal keys inside one lane need the run bookkeeping (with a ragged last lane the -inf fillers do not count)
  bool lane_dup = false;
#pragma unroll
  for (int v = 0; v + 1 < VPL; ++v) lane_dup |= (key[v] == key[v + 1]) && (FULL || key[v] > KEY_NEG_INF);
  const bool any_dup = __any_sync(0xffffffffu, lane_dup);
  uint32_t head = key[0];

  // ---- group selection: a group's score is the sum of its two best choices ----
  if (LG >= 0 || p.n_group > 1) {
    const int lg = LG >= 0 ? LG : p.lanes_per_group_log2;   // a group spans 2^lg lanes
    const int lpg = 1 << lg;
    const int n_group = LG >= 0 ? (32 >> LG) : p.n_group;
    float t1 = f[0];
    float t2 = -CUDART_INF_F;
    if constexpr (VPL >= 2) t2 = f[1];
#pragma unroll
    for (int o = 1; o < lpg; o <<= 1) {
      const float o1 = __shfl_xor_sync(0xffffffffu, t1, o);
      const float o2 = __shfl_xor_sync(0xffffffffu, t2, o);
      merge_top2(t1, t2, o1, o2);
    }
    const int my_group = lane >> lg;
    const float my_score = (LG >= 0 || my_group < n_group) ? __fadd_rn(t1, t2) : -CUDART_INF_F;
    // rank = groups that beat mine (ties: lower index).  The lanes of a group share the comparisons:
    // each takes a slice of the groups, then the partial counts are summed inside the group.
    const int per = (n_group + lpg - 1) >> lg;
    const int g0 = (lane & (lpg - 1)) * per;
    int rank = 0;
#pragma unroll
    for (int i = 0; i < per; ++i) {
      const int g = g0 + i;
      const float gs = __shfl_sync(0xffffffffu, my_score, (g << lg) & 31);
      rank += (g < n_group) && ((gs > my_score) || (gs == my_score && g < my_group));
    }
#pragma unroll
    for (int o = 1; o < lpg; o <<= 1) rank += __shfl_xor_sync(0xffffffffu, rank, o);
    // a lane of a dropped group retires: top_k never exceeds the experts of the kept groups (checked by the
    // entry point), so its list is never needed
    head = ((LG >= 0 || my_group < n_group) && (rank < p.topk_group)) ? head : 0u;
  }

  // ---- top-k (ties -> lower expert index) ----
  uint2* win = sm_win[threadIdx.x >> 5];
  const int top_k = TOPK > 0 ? TOPK : p.top_k;
  if (!any_dup) topk_rounds<false, TOPK>(head, my_list, win, top_k, lane);
  else topk_rounds<true, TOPK>(head, my_list, win, top_k, lane);
  __syncwarp();
  const uint2 mine = win[lane < top_k ? lane : 0];
  const uint32_t my_key = mine.x;
  const int my_owner = mine.y & 0xff, my_dup = mine.y >> 8;
  int my_v = 0;
  {
    const uint32_t* ok = wkeys + my_owner * VPL;
    uint32_t orig[VPL];
    if constexpr (VPL >= 4) {
#pragma unroll
      for (int v = 0; v < VPL; v += 4) {
        const uint4 q = *reinterpret_cast<const uint4*>(ok + v);
        orig[v] = q.x; orig[v + 1] = q.y; orig[v + 2] = q.z; orig[v + 3] = q.w;
      }
    } else {
#pragma unroll
      for (int v = 0; v < VPL; ++v) orig[v] = ok[v];
    }
#pragma unroll
    for (int v = VPL - 1; v >= 0; --v) my_v = (orig[v] == my_key) ? v : my_v;
    if (any_dup) {     // take the (run+1)-th match
      int seen = 0, pick = my_v;
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        const bool m = orig[v] == my_key;
        if (m && seen == my_dup) pick = v;
        seen += m;
      }
      my_v = pick;
    }
  }
  const int my_id = my_owner * VPL + my_v;
  const float my_w = (lane < top_k) ? wscores[my_id] : 0.f;
  float wsum = my_w;
  // lanes >= top_k hold 0, so with top_k <= 8 the first two levels of the tree add exact zeros and are skipped
#pragma unroll
  for (int o = (TOPK > 0 && TOPK <= 8) ? 4 : 16; o > 0; o >>= 1) wsum += __shfl_xor_sync(0xffffffffu, wsum, o);
  if (lane < top_k) {
    float w = my_w;
    if (p.renormalize) w = __fdividef(w, wsum + 1e-20f);
    w *= p.scale;
    p.ids[token * top_k + lane] = my_id;
    p.weights[token * top_k + lane] = w;
  }
}

// Launch the one-warp-per-token router for prepared parameters.
static int launch_gating(const GatingParams& p_in, void* stream) {
  GatingParams p = p_in;
  int vpl = 1;
  while (vpl * 32 < p.experts) vpl <<= 1;
  p.lanes_per_group = 1;
  p.lanes_per_group_log2 = 0;
  if (p.n_group > 1) {
    p.lanes_per_group = (p.experts / p.n_group) / vpl;     // power of two, checked by the caller
    while ((1 << p.lanes_per_group_log2) < p.lanes_per_group) ++p.lanes_per_group_log2;
  }
  const bool full = p.experts == 32 * vpl && ((uintptr_t)p.logits & 15) == 0 && (p.ld % 4) == 0 &&
                    ((uintptr_t)p.bias & 15) == 0;
  const int warps = vpl >= 16 ? 4 : 8;                     // GateShape<VPL>::WARPS
  const int64_t blocks = (p.tokens + warps - 1) / warps;
  DLB_CHECK_ARG(blocks <= 0x7fffffffLL, DLB_ERR_TOO_LARGE, "gating: too many tokens");
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned g = (unsigned)blocks, t = warps * 32;
  switch (vpl) {
    case 1: grouped_topk_kernel<1, false><<<g, t, 0, s>>>(p); break;
    case 2: grouped_topk_kernel<2, false><<<g, t, 0, s>>>(p); break;
    case 4:
      if (full) grouped_topk_kernel<4, true><<<g, t, 0, s>>>(p);
      else grouped_topk_kernel<4, false><<<g, t, 0, s>>>(p);
      break;
    case 8:
      if (full && p.n_group == 8 && p.top_k == 8 && p.scoring == DLB_SCORE_SIGMOID)
        grouped_topk_kernel<8, true, 2, 8><<<g, t, 0, s>>>(p);
      else if (full) grouped_topk_kernel<8, true><<<g, t, 0, s>>>(p);
      else grouped_topk_kernel<8, false><<<g, t, 0, s>>>(p);
      break;
    default:
      if (full) grouped_topk_kernel<16, true><<<g, t, 0, s>>>(p);
      else grouped_topk_kernel<16, false><<<g, t, 0, s>>>(p);
      break;
  }
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

// ----------------------------------------------------------------------------
// GShard-style top-k gating with capacity (the reference's `topk_gating` family,
// python/dlBLAS/dlblas/kernels/topk_gating.py:259-290 and topk_gating_fwd_part1/2/3.py;
// torch statement in python/dlBLAS/benchmarks/topk_gating.py:132-206).
//   gates = softmax(logits); the k choices of every token queue up per expert in
//   (choice-major, token) order; a choice is kept if its queue position is below the
//   capacity; weights = kept gate values normalised over the token's kept choices.
// Queue positions come from the stable counting sort of moe_align (block 1) over the
// choice-major id list, so no [k, S, E] mask tensors are materialised.
// ----------------------------------------------------------------------------
// Deterministic column sums of gates [S, E]: stage 1 reduces row chunks, stage 2 the partials.
__global__ void __launch_bounds__(256) gshard_colsum_stage1(const float* __restrict__ gates, float* __restrict__ part,
                                                            int64_t S, int E, int rows_per_block) {
  const int64_t r0 = (int64_t)blockIdx.x * rows_per_block;
  const int64_t r1 = min(S, r0 + rows_per_block);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float acc = 0.f;
    for (int64_t r = r0; r < r1; ++r) acc += gates[r * E + e];
    part[(int64_t)blockIdx.x * E + e] = acc;
  }
}
// me[e] = sum / S;  ce[e] = first-choice count / S;  l_aux = mean(me * ce) * E * E
__global__ void __launch_bounds__(256) gshard_aux_kernel(const float* __restrict__ part, int nblk,
                                                         const int32_t* __restrict__ ids_km /* [K*S] */,
                                                         int64_t S, int E, float* __restrict__ me,
                                                         float* __restrict__ ce, float* __restrict__ l_aux) {
  extern __shared__ float sh[];   // [E] first-choice counts, then reduction scratch
  float* cnt = sh;
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0.f;
  __syncthreads();
  for (int64_t i = threadIdx.x; i < S; i += blockDim.x) atomicAdd(&cnt[ids_km[i]], 1.0f);   // integers: exact
  __syncthreads();
  float local = 0.f;
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    float acc = 0.f;
    for (int b = 0; b < nblk; ++b) acc += part[(int64_t)b * E + e];
    const float m = acc / (float)S, c = cnt[e] / (float)S;
    me[e] = m;
    ce[e] = c;
    local += m * c;
  }
  __shared__ float red[8];
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) local += __shfl_xor_sync(0xffffffffu, local, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = local;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) t += red[w];
    l_aux[0] = t / (float)E * (float)E * (float)E;
  }
}
// Queue position of every (choice, token) slot and the per-expert token lists.
__global__ void __launch_bounds__(256) gshard_queue_kernel(const int32_t* __restrict__ sorted_slots,
                                                           const int32_t* __restrict__ prefix,
                                                           const int32_t* __restrict__ ids_km,
                                                           int32_t* __restrict__ loc, int64_t* __restrict__ select,
                                                           int64_t KS, int64_t S, int E, int capacity) {
  for (int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < KS; p += (int64_t)gridDim.x * blockDim.x) {
    const int slot = sorted_slots[p];
    const int e = ids_km[slot];
    const int l = (int)p - prefix[e];
    loc[slot] = l;
    if (l < capacity) select[(int64_t)e * capacity + l] = slot % S;   // token of the l-th kept choice
  }
}
// Capacity slots no choice filled are given the lowest-numbered tokens that did not choose the expert
// within capacity; they carry no weight (the reference fills them with arbitrary zero-valued tokens).
__global__ void __launch_bounds__(256) gshard_fill_kernel(const int32_t* __restrict__ prefix,
                                                          int64_t* __restrict__ select, int E, int capacity,
                                                          int64_t S) {
  const int e = blockIdx.x;
  const int kept = min(prefix[e + 1] - prefix[e], capacity);
  // the kept tokens of this expert, as a bitmap in shared memory
  extern __shared__ uint32_t bits[];
  const int words = (int)((S + 31) / 32);
  for (int w = threadIdx.x; w < words; w += blockDim.x) bits[w] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < kept; i += blockDim.x) {
    const int64_t t = select[(int64_t)e * capacity + i];
    atomicOr(&bits[t >> 5], 1u << (t & 31));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int out = kept;
    for (int64_t t = 0; t < S && out < capacity; ++t)
      if (!((bits[t >> 5] >> (t & 31)) & 1u)) select[(int64_t)e * capacity + out++] = t;
  }
}
// Per token: drop choices beyond capacity, normalise the kept gate values, emit e * capacity + position.
__global__ void __launch_bounds__(256) gshard_assign_kernel(const float* __restrict__ gates,
                                                            const int32_t* __restrict__ ids_km,
                                                            const int32_t* __restrict__ loc,
                                                            int32_t* __restrict__ ec_idx, float* __restrict__ weights,
                                                            int64_t S, int E, int K, int capacity, float eps) {
  const int64_t s = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= S) return;
  float denom = 0.f;
  for (int k = 0; k < K; ++k) {
    const int e = ids_km[k * S + s];
    if (loc[k * S + s] < capacity) denom += gates[s * E + e];
  }
  denom = fmaxf(denom, eps);
  for (int k = 0; k < K; ++k) {
    const int e = ids_km[k * S + s];
    const int l = loc[k * S + s];
    const bool kept = l < capacity;
    const float g = kept ? gates[s * E + e] : 0.f;
    weights[k * S + s] = g / denom;
    ec_idx[k * S + s] = kept && g > 0.f ? e * capacity + l : (kept ? l : 0);
  }
}
// grad_logits[s, i] = g_i * (gg_i - sum_j g_j gg_j),  gg_e = grad_l_aux * ce[e] * E / S
// (python/dlBLAS/dlblas/kernels/topk_gating_bwd.py:20-66)
__global__ void __launch_bounds__(256) gshard_bwd_kernel(const float* __restrict__ gates, const float* __restrict__ ce,
                                                         const float* __restrict__ grad_l_aux,
                                                         float* __restrict__ grad_logits, int64_t S, int E) {
  const int lane = threadIdx.x & 31;
  const int64_t s = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (s >= S) return;
  const float scale = grad_l_aux[0] * (float)E / (float)S;
  float dot = 0.f;
  for (int e = lane; e < E; e += 32) dot += gates[s * E + e] * (ce[e] * scale);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  for (int e = lane; e < E; e += 32) {
    const float g = gates[s * E + e];
    grad_logits[s * E + e] = g * (ce[e] * scale - dot);
  }
}

// Backward through the routing weights as well (the reference's `higher_precision` path,
// python/dlBLAS/dlblas/kernels/topk_gating.py:145-256): with g_k the kept gate values of a token,
// D = sum_k g_k, C = max(D, eps) and w_k = g_k / C,
//   d loss / d g_k = gw_k / C - [D >= eps] * sum_j gw_j g_j / C^2        (kept choices only)
// is scattered to the chosen experts, the auxiliary-loss term grad_l_aux * ce[e] * E / S is added, and
// the result goes through the softmax backward  grad_logits_i = g_i * (gg_i - sum_j g_j gg_j).
// One warp per token; lane k < K holds choice k.
__global__ void __launch_bounds__(256) gshard_bwd_weights_kernel(
    const float* __restrict__ gates, const float* __restrict__ ce, const float* __restrict__ grad_l_aux,
    const int32_t* __restrict__ ids_km, const int32_t* __restrict__ loc, const float* __restrict__ grad_weights,
    float* __restrict__ grad_logits, int64_t S, int E, int K, int capacity, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t s = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (s >= S) return;
  const float scale = grad_l_aux[0] * (float)E / (float)S;
  int my_e = -1;
  float my_g = 0.f, my_gw = 0.f;
  if (lane < K) {
    const int e = ids_km[(int64_t)lane * S + s];
    if (loc[(int64_t)lane * S + s] < capacity) {
      my_e = e;
      my_g = gates[s * E + e];
      my_gw = grad_weights[(int64_t)lane * S + s];
    }
  }
  float denom = my_g, cross = my_gw * my_g;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    denom += __shfl_xor_sync(0xffffffffu, denom, o);
    cross += __shfl_xor_sync(0xffffffffu, cross, o);
  }
  const float c = fmaxf(denom, eps);
  const float common = denom >= eps ? -cross / (c * c) : 0.f;
  const float my_d = my_e >= 0 ? my_gw / c + common : 0.f;     // d loss / d gate of my choice
  float dot = 0.f;
  for (int e0 = 0; e0 < E; e0 += 32) {
    const int e = e0 + lane;
    float gg = e < E ? ce[e] * scale : 0.f;
    for (int k = 0; k < K; ++k) {
      const int ek = __shfl_sync(0xffffffffu, my_e, k);
      const float dk = __shfl_sync(0xffffffffu, my_d, k);
      if (ek == e) gg += dk;
    }
    if (e < E) dot += gates[s * E + e] * gg;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
  for (int e0 = 0; e0 < E; e0 += 32) {
    const int e = e0 + lane;
    float gg = e < E ? ce[e] * scale : 0.f;
    for (int k = 0; k < K; ++k) {
      const int ek = __shfl_sync(0xffffffffu, my_e, k);
      const float dk = __shfl_sync(0xffffffffu, my_d, k);
      if (ek == e) gg += dk;
    }
    if (e < E) grad_logits[s * E + e] = gates[s * E + e] * (gg - dot);
  }
}

}  // namespace dlb

extern "C" int dlb_grouped_topk_gating(const float* logits, const float* bias, int32_t* ids, float* weights,
                                       int64_t tokens, int experts, int64_t logits_row_stride, int n_group,
                                       int topk_group, int top_k, int scoring, int renormalize, float scale,
                                       void* stream) {
  DLB_NVTX("dlb_grouped_topk_gating");
  using namespace dlb;
  DLB_CHECK_ARG(tokens >= 0, DLB_ERR_BAD_ARG, "gating: negative token count");
  DLB_CHECK_ARG(experts >= 1 && experts <= 512, DLB_ERR_UNSUPPORTED, "gating: experts=%d not in [1, 512]", experts);
  DLB_CHECK_ARG(top_k >= 1 && top_k <= 32 && top_k <= experts, DLB_ERR_BAD_ARG, "gating: top_k=%d invalid", top_k);
  DLB_CHECK_ARG(scoring == DLB_SCORE_SIGMOID || scoring == DLB_SCORE_SOFTMAX, DLB_ERR_BAD_ARG,
                "gating: scoring=%d invalid", scoring);
  DLB_CHECK_ARG(n_group >= 1 && topk_group >= 1 && topk_group <= n_group, DLB_ERR_BAD_ARG,
                "gating: n_group=%d topk_group=%d invalid", n_group, topk_group);
  DLB_CHECK_ARG(logits_row_stride >= experts, DLB_ERR_BAD_ARG, "gating: row stride smaller than experts");
  if (tokens == 0) return DLB_OK;
  DLB_CHECK_ARG(logits && ids && weights, DLB_ERR_BAD_ARG, "gating: null pointer");

  int vpl = 1;
  while (vpl * 32 < experts) vpl <<= 1;
  if (n_group > 1) {
    DLB_CHECK_ARG(experts % n_group == 0, DLB_ERR_BAD_ARG, "gating: experts %% n_group != 0");
    const int gs = experts / n_group;
    DLB_CHECK_ARG(gs % vpl == 0, DLB_ERR_UNSUPPORTED, "gating: group size %d not a multiple of %d lanes-worth", gs,
                  vpl);
    const int lpg = gs / vpl;
    DLB_CHECK_ARG((lpg & (lpg - 1)) == 0 && lpg <= 32, DLB_ERR_UNSUPPORTED,
                  "gating: group must span a power-of-two number of lanes (got %d)", lpg);
    DLB_CHECK_ARG(top_k <= topk_group * gs, DLB_ERR_BAD_ARG, "gating: top_k exceeds experts in kept groups");
    DLB_CHECK_ARG(gs >= 2, DLB_ERR_BAD_ARG, "gating: groups need at least two experts");
  }
  // 128-bit loads need 16-byte aligned rows
  if (vpl >= 4) {
    DLB_CHECK_ARG(((uintptr_t)logits & 15) == 0 && (logits_row_stride % 4) == 0, DLB_ERR_ALIGNMENT,
                  "gating: logits rows must be 16-byte aligned");
  }
  GatingParams p{logits, bias, ids, weights, nullptr, tokens, logits_row_stride, experts, n_group,
                 topk_group, top_k, scoring, renormalize, scale};
  return launch_gating(p, stream);
}


extern "C" int dlb_gshard_gate(const float* logits, int64_t tokens, int experts, int top_k, float* gates,
                               int32_t* ids /* [tokens, top_k] */, float* scratch_weights, void* stream) {
  DLB_NVTX("dlb_gshard_gate");
  using namespace dlb;
  DLB_CHECK_ARG(tokens >= 0 && experts >= 1 && experts <= 512 && top_k >= 1 && top_k <= 32 && top_k <= experts,
                DLB_ERR_BAD_ARG, "gshard_gate: bad sizes");
  if (tokens == 0) return DLB_OK;
  DLB_CHECK_ARG(logits && gates && ids && scratch_weights, DLB_ERR_BAD_ARG, "gshard_gate: null pointer");
  int vpl = 1;
  while (vpl * 32 < experts) vpl <<= 1;
  if (vpl >= 4)
    DLB_CHECK_ARG(((uintptr_t)logits & 15) == 0 && experts % 4 == 0, DLB_ERR_ALIGNMENT,
                  "gshard_gate: logits rows must be 16-byte aligned");
  GatingParams p{logits, nullptr, ids, scratch_weights, gates, tokens, experts, experts, 1, 1, top_k,
                 DLB_SCORE_SOFTMAX, 0, 1.0f};
  return launch_gating(p, stream);
}

extern "C" int dlb_gshard_assign(const float* gates, const int32_t* ids_choice_major, const int32_t* sorted_slots,
                                 const int32_t* expert_prefix, int64_t tokens, int experts, int top_k,
                                 int64_t capacity, float* colsum_scratch, int64_t colsum_blocks, int32_t* loc,
                                 float* me, float* ce, float* l_aux, int32_t* ec_idx, float* weights,
                                 int64_t* expert_select_token_idx, void* stream) {
  DLB_NVTX("dlb_gshard_assign");
  using namespace dlb;
  DLB_CHECK_ARG(tokens >= 1 && experts >= 1 && experts <= 1024 && top_k >= 1 && capacity >= 1 && colsum_blocks >= 1,
                DLB_ERR_BAD_ARG, "gshard_assign: bad sizes");
  DLB_CHECK_ARG(tokens * top_k < (1LL << 31) && (int64_t)experts * capacity < (1LL << 31), DLB_ERR_TOO_LARGE,
                "gshard_assign: problem too large");
  DLB_CHECK_ARG(gates && ids_choice_major && sorted_slots && expert_prefix && colsum_scratch && loc && me && ce &&
                    l_aux && ec_idx && weights && expert_select_token_idx,
                DLB_ERR_BAD_ARG, "gshard_assign: null pointer");
  cudaStream_t s = (cudaStream_t)stream;
  const int rows_per_block = (int)((tokens + colsum_blocks - 1) / colsum_blocks);
  gshard_colsum_stage1<<<(unsigned)colsum_blocks, 256, 0, s>>>(gates, colsum_scratch, tokens, experts, rows_per_block);
  DLB_CUDA_LAUNCH_CHECK();
  gshard_aux_kernel<<<1, 256, experts * sizeof(float), s>>>(colsum_scratch, (int)colsum_blocks, ids_choice_major,
                                                            tokens, experts, me, ce, l_aux);
  DLB_CUDA_LAUNCH_CHECK();
  const int64_t KS = tokens * top_k;
  int64_t blocks = (KS + 255) / 256;
  if (blocks > 4096) blocks = 4096;
  gshard_queue_kernel<<<(unsigned)blocks, 256, 0, s>>>(sorted_slots, expert_prefix, ids_choice_major, loc,
                                                       expert_select_token_idx, KS, tokens, experts, (int)capacity);
  DLB_CUDA_LAUNCH_CHECK();
  const size_t bitmap = (size_t)((tokens + 31) / 32) * 4;
  DLB_CHECK_ARG(bitmap <= 200 * 1024, DLB_ERR_TOO_LARGE, "gshard_assign: more than 1.6M tokens");
  cudaError_t e = cudaFuncSetAttribute(gshard_fill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bitmap);
  if (e != cudaSuccess) {
    set_last_error("gshard_assign: smem attribute: %s", cudaGetErrorString(e));
    return (int)e;
  }
  gshard_fill_kernel<<<(unsigned)experts, 256, bitmap, s>>>(expert_prefix, expert_select_token_idx, experts,
                                                            (int)capacity, tokens);
  DLB_CUDA_LAUNCH_CHECK();
  gshard_assign_kernel<<<(unsigned)((tokens + 255) / 256), 256, 0, s>>>(gates, ids_choice_major, loc, ec_idx, weights,
                                                                        tokens, experts, top_k, (int)capacity,
                                                                        1.1920928955078125e-07f);
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

extern "C" int dlb_gshard_gate_bwd(const float* gates, const float* ce, const float* grad_l_aux, float* grad_logits,
                                   int64_t tokens, int experts, void* stream) {
  DLB_NVTX("dlb_gshard_gate_bwd");
  using namespace dlb;
  DLB_CHECK_ARG(tokens >= 0 && experts >= 1, DLB_ERR_BAD_ARG, "gshard_gate_bwd: bad sizes");
  if (tokens == 0) return DLB_OK;
  DLB_CHECK_ARG(gates && ce && grad_l_aux && grad_logits, DLB_ERR_BAD_ARG, "gshard_gate_bwd: null pointer");
  const int64_t blocks = (tokens + 7) / 8;
  DLB_CHECK_ARG(blocks <= 0x7fffffffLL, DLB_ERR_TOO_LARGE, "gshard_gate_bwd: too many tokens");
  gshard_bwd_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(gates, ce, grad_l_aux, grad_logits, tokens,
                                                                        experts);
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

extern "C" int dlb_gshard_gate_bwd_weights(const float* gates, const float* ce, const float* grad_l_aux,
                                           const int32_t* ids_choice_major, const int32_t* loc,
                                           const float* grad_weights, float* grad_logits, int64_t tokens, int experts,
                                           int top_k, int64_t capacity, void* stream) {
  DLB_NVTX("dlb_gshard_gate_bwd_weights");
  using namespace dlb;
  DLB_CHECK_ARG(tokens >= 0 && experts >= 1 && top_k >= 1 && top_k <= 32 && capacity >= 1, DLB_ERR_BAD_ARG,
                "gshard_gate_bwd_weights: bad sizes");
  if (tokens == 0) return DLB_OK;
  DLB_CHECK_ARG(gates && ce && grad_l_aux && ids_choice_major && loc && grad_weights && grad_logits, DLB_ERR_BAD_ARG,
                "gshard_gate_bwd_weights: null pointer");
  DLB_CHECK_ARG(capacity < (1LL << 31), DLB_ERR_TOO_LARGE, "gshard_gate_bwd_weights: capacity too large");
  const int64_t blocks = (tokens + 7) / 8;
  DLB_CHECK_ARG(blocks <= 0x7fffffffLL, DLB_ERR_TOO_LARGE, "gshard_gate_bwd_weights: too many tokens");
  gshard_bwd_weights_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      gates, ce, grad_l_aux, ids_choice_major, loc, grad_weights, grad_logits, tokens, experts, top_k, (int)capacity,
      1.1920928955078125e-07f);
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}
