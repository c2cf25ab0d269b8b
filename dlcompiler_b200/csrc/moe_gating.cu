// MoE router: grouped top-k gating (DeepSeek-V3 style) and plain softmax top-k.
//
// One warp per token.  Lane l owns the VPL consecutive experts
// [l*VPL, (l+1)*VPL), loaded as 128-bit vectors; every reduction (softmax
// max/sum, per-group top-2 sums, group ranking, k rounds of arg-max) is a
// warp-shuffle tree, so no shared memory and no atomics are used and the
// result is deterministic.
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
  int64_t tokens;
  int64_t ld;
  int experts;
  int n_group;
  int topk_group;
  int top_k;
  int scoring;
  int renormalize;
  float scale;
};

// sigmoid evaluated by a FIXED sequence of correctly-rounded fp32 operations
// (no fused multiply-add, no approximate transcendental), so that the CPU checker,
// which performs the same sequence with IEEE fp32 tensor ops, gets bit-identical
// scores and therefore bit-identical expert ids even for near-ties:
//   t = clamp(-x, -87, 88); n = rint(t * log2e); r = (t - n*LN2_HI) - n*LN2_LO
//   e = (((((r/720 + 1/120) r + 1/24) r + 1/6) r + 1/2) r + 1) r + 1   [Horner]
//   sigmoid = 1 / (1 + e * 2^n)
__device__ __forceinline__ float sigmoid_spec(float x) {
  const float t = fminf(fmaxf(-x, -87.0f), 88.0f);
  const float n = rintf(__fmul_rn(t, 1.44269502162933349609375f));
  float r = __fsub_rn(t, __fmul_rn(n, 0.693145751953125f));
  r = __fsub_rn(r, __fmul_rn(n, 1.428606765330187045037746429443359375e-06f));
  float p = 1.38888892251998186111450195312e-03f;                 // 1/720
  p = __fadd_rn(__fmul_rn(p, r), 8.33333376795053482055664062500e-03f);   // 1/120
  p = __fadd_rn(__fmul_rn(p, r), 4.16666679084300994873046875000e-02f);   // 1/24
  p = __fadd_rn(__fmul_rn(p, r), 1.66666671633720397949218750000e-01f);   // 1/6
  p = __fadd_rn(__fmul_rn(p, r), 0.5f);
  p = __fadd_rn(__fmul_rn(p, r), 1.0f);
  p = __fadd_rn(__fmul_rn(p, r), 1.0f);
  const float two_n = __int_as_float(((int)n + 127) << 23);
  const float e = __fmul_rn(p, two_n);
  return __frcp_rn(__fadd_rn(1.0f, e));
}

__device__ __forceinline__ void merge_top2(float& a1, float& a2, float b1, float b2) {
  // (a1 >= a2), (b1 >= b2) -> two largest of the four
  const float hi = fmaxf(a1, b1);
  const float lo = fmaxf(fminf(a1, b1), fmaxf(a2, b2));
  a1 = hi;
  a2 = lo;
}

template <int VPL>
__global__ void __launch_bounds__(256) grouped_topk_kernel(GatingParams p) {
  const int lane = threadIdx.x & 31;
  const int warps_per_block = blockDim.x >> 5;
  const int64_t token = (int64_t)blockIdx.x * warps_per_block + (threadIdx.x >> 5);
  if (token >= p.tokens) return;  // whole warp leaves together

  const int E = p.experts;
  const int e0 = lane * VPL;
  const float* row = p.logits + token * p.ld;

  float s[VPL];  // un-biased score (sigmoid or softmax probability)
  float c[VPL];  // selection score
  // ---- load ----
  if constexpr (VPL >= 4) {
#pragma unroll
    for (int v = 0; v < VPL; v += 4) {
      if (e0 + v + 3 < E) {
        const float4 x = __ldg(reinterpret_cast<const float4*>(row + e0 + v));
        s[v] = x.x; s[v + 1] = x.y; s[v + 2] = x.z; s[v + 3] = x.w;
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) s[v + j] = (e0 + v + j < E) ? __ldg(row + e0 + v + j) : -CUDART_INF_F;
      }
    }
  } else {
#pragma unroll
    for (int v = 0; v < VPL; ++v) s[v] = (e0 + v < E) ? __ldg(row + e0 + v) : -CUDART_INF_F;
  }

  // ---- scoring ----
  if (p.scoring == DLB_SCORE_SIGMOID) {
#pragma unroll
    for (int v = 0; v < VPL; ++v) s[v] = (e0 + v < E) ? sigmoid_spec(s[v]) : -CUDART_INF_F;
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
      s[v] = (e0 + v < E) ? expf(s[v] - m) : 0.f;
      sum += s[v];
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
#pragma unroll
    for (int v = 0; v < VPL; ++v) s[v] = (e0 + v < E) ? s[v] / sum : -CUDART_INF_F;
  }
  if (p.scoring == DLB_SCORE_SIGMOID || p.bias != nullptr) {
#pragma unroll
    for (int v = 0; v < VPL; ++v) {
      const bool valid = e0 + v < E;
      c[v] = valid ? (p.bias != nullptr ? __fadd_rn(s[v], __ldg(p.bias + e0 + v)) : s[v]) : -CUDART_INF_F;
    }
  }

  // ---- group selection ----
  if (p.n_group > 1) {
    const int lanes_per_group = (E / p.n_group) / VPL;  // power of two, checked on the host
    float t1 = -CUDART_INF_F, t2 = -CUDART_INF_F;
#pragma unroll
    for (int v = 0; v < VPL; ++v) merge_top2(t1, t2, c[v], -CUDART_INF_F);
    for (int o = 1; o < lanes_per_group; o <<= 1) {
      const float o1 = __shfl_xor_sync(0xffffffffu, t1, o);
      const float o2 = __shfl_xor_sync(0xffffffffu, t2, o);
      merge_top2(t1, t2, o1, o2);
    }
    const int my_group = lane / lanes_per_group;
    const float my_score = (my_group < p.n_group) ? __fadd_rn(t1, t2) : -CUDART_INF_F;
    int rank = 0;
    for (int g = 0; g < p.n_group; ++g) {
      const float gs = __shfl_sync(0xffffffffu, my_score, g * lanes_per_group);
      rank += (gs > my_score) || (gs == my_score && g < my_group);
    }
    const bool keep = (my_group < p.n_group) && (rank < p.topk_group);
    if (!keep) {
#pragma unroll
      for (int v = 0; v < VPL; ++v) c[v] = -CUDART_INF_F;
    }
  }

  // ---- top-k: k rounds of warp arg-max (ties -> lower expert index) ----
  // Scores become order-preserving unsigned keys so that one hardware warp reduction
  // (redux.sync) finds the maximum; a second one picks the lowest expert index among equals.
  // Each lane caches its local best; only the winning lane rescans after a round.
  uint32_t key[VPL];
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    const uint32_t b = __float_as_uint(c[v]);
    key[v] = (b & 0x80000000u) ? ~b : (b | 0x80000000u);      // -inf maps to 0x007fffff: below every finite score
  }
  uint32_t lbest = 0;
  int lidx = 0;
#pragma unroll
  for (int v = 0; v < VPL; ++v) {
    if (key[v] > lbest) {   // strict: the lower index wins a tie inside the lane
      lbest = key[v];
      lidx = v;
    }
  }
  float wsum = 0.f;
  float my_w = 0.f;   // lane i < K keeps weight i
  int my_id = 0;
  for (int k = 0; k < p.top_k; ++k) {
    const uint32_t wmax = __reduce_max_sync(0xffffffffu, lbest);
    const int cand = (lbest == wmax) ? e0 + lidx : 0x7fffffff;
    const int best_e = __reduce_min_sync(0xffffffffu, cand);
    const int owner = best_e / VPL;
    float ls = 0.f;
#pragma unroll
    for (int v = 0; v < VPL; ++v)
      if (v == lidx) ls = s[v];
    const float best_s = __shfl_sync(0xffffffffu, ls, owner);
    if (lane == owner) {
      // retire the winner and rescan this lane only
#pragma unroll
      for (int v = 0; v < VPL; ++v)
        if (v == lidx) key[v] = 0;
      lbest = 0;
      lidx = 0;
#pragma unroll
      for (int v = 0; v < VPL; ++v) {
        if (key[v] > lbest) {
          lbest = key[v];
          lidx = v;
        }
      }
    }
    wsum += best_s;
    if (lane == k) {
      my_w = best_s;
      my_id = best_e;
    }
  }
  if (lane < p.top_k) {
    float w = my_w;
    if (p.renormalize) w = w / (wsum + 1e-20f);
    w *= p.scale;
    p.ids[token * p.top_k + lane] = my_id;
    p.weights[token * p.top_k + lane] = w;
  }
}

}  // namespace dlb

extern "C" int dlb_grouped_topk_gating(const float* logits, const float* bias, int32_t* ids, float* weights,
                                       int64_t tokens, int experts, int64_t logits_row_stride, int n_group,
                                       int topk_group, int top_k, int scoring, int renormalize, float scale,
                                       void* stream) {
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
  GatingParams p{logits, bias, ids, weights, tokens, logits_row_stride, experts, n_group,
                 topk_group, top_k, scoring, renormalize, scale};
  const int warps = 8;
  const int64_t blocks = (tokens + warps - 1) / warps;
  DLB_CHECK_ARG(blocks <= 0x7fffffffLL, DLB_ERR_TOO_LARGE, "gating: too many tokens");
  cudaStream_t s = (cudaStream_t)stream;
  switch (vpl) {
    case 1: grouped_topk_kernel<1><<<(unsigned)blocks, warps * 32, 0, s>>>(p); break;
    case 2: grouped_topk_kernel<2><<<(unsigned)blocks, warps * 32, 0, s>>>(p); break;
    case 4: grouped_topk_kernel<4><<<(unsigned)blocks, warps * 32, 0, s>>>(p); break;
    case 8: grouped_topk_kernel<8><<<(unsigned)blocks, warps * 32, 0, s>>>(p); break;
    default: grouped_topk_kernel<16><<<(unsigned)blocks, warps * 32, 0, s>>>(p); break;
  }
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}
