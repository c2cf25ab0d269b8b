// moe_align_block_size, row permute (gather) and top-k combine for fused_moe.
//
// moe_align_block_size is the block-padded form of the reference's
// argsort + per-expert [start, end) ranges
// (python/dlBLAS/dlblas/kernels/fused_moe.py:238-293, 314-320):
//   * the (token, k) slots 0..numel-1 are counting-sorted by expert id, stable
//     (ascending slot index inside an expert),
//   * every expert segment is padded to a multiple of `block` with the
//     sentinel value `numel`,
//   * expert_ids[b] is the expert that owns block b of the padded list,
//   * num_tokens_post_padded[0] is the padded length,
//   * block_start[e] (E + 1 entries) is the first block of expert e.
// Slots whose id is outside [0, E) (experts owned by another rank) are dropped.
// All outputs are integer and bit-exact reproducible: positions are derived
// from prefix sums and warp match masks, never from atomics on positions.
#include "common.cuh"

namespace dlb {

constexpr int ALIGN_THREADS = 1024;
constexpr int ALIGN_WARPS = ALIGN_THREADS / 32;

template <typename IdT>
__global__ void __launch_bounds__(ALIGN_THREADS) moe_align_kernel(
    const IdT* __restrict__ topk_ids, int32_t* __restrict__ sorted_token_ids, int32_t* __restrict__ expert_ids,
    int32_t* __restrict__ num_tokens_post_padded, int32_t* __restrict__ block_start, int numel, int num_experts,
    int block, int sorted_capacity, int expert_ids_capacity) {
  extern __shared__ int32_t smem[];
  int32_t* counts = smem;                          // [E]    tokens per expert
  int32_t* seg_off = counts + num_experts;         // [E+1]  padded start of each expert
  int32_t* running = seg_off + num_experts + 1;    // [E]    tokens already placed per expert
  int32_t* warp_cnt = running + num_experts;       // [ALIGN_WARPS][E]
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int warp = tid >> 5;

  for (int e = tid; e < num_experts; e += ALIGN_THREADS) {
    counts[e] = 0;
    running[e] = 0;
  }
  __syncthreads();
  // 1. histogram (integer adds commute, so shared atomics stay deterministic)
  for (int i = tid; i < numel; i += ALIGN_THREADS) {
    const int64_t e = (int64_t)topk_ids[i];
    if (e >= 0 && e < num_experts) atomicAdd(&counts[(int)e], 1);
  }
  __syncthreads();
  // 2. exclusive scan of the padded counts (serial over experts: E <= 1024)
  if (tid == 0) {
    int acc = 0;
    int blk = 0;
    for (int e = 0; e < num_experts; ++e) {
      seg_off[e] = acc;
      block_start[e] = blk;
      const int nb = (counts[e] + block - 1) / block;
      for (int b = 0; b < nb; ++b)
        if (blk + b < expert_ids_capacity) expert_ids[blk + b] = e;
      blk += nb;
      acc += nb * block;
    }
    seg_off[num_experts] = acc;
    block_start[num_experts] = blk;
    num_tokens_post_padded[0] = acc;
    for (int b = blk; b < expert_ids_capacity; ++b) expert_ids[b] = -1;
  }
  // 3. sentinel fill of the whole capacity
  for (int i = tid; i < sorted_capacity; i += ALIGN_THREADS) sorted_token_ids[i] = numel;
  __syncthreads();
  // 4. stable placement, ALIGN_THREADS consecutive slots per round
  for (int base = 0; base < numel; base += ALIGN_THREADS) {
    for (int i = tid; i < ALIGN_WARPS * num_experts; i += ALIGN_THREADS) warp_cnt[i] = 0;
    __syncthreads();
    const int slot = base + tid;
    int e = -1;
    if (slot < numel) {
      const int64_t v = (int64_t)topk_ids[slot];
      if (v >= 0 && v < num_experts) e = (int)v;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && rank_in_warp == 0) warp_cnt[warp * num_experts + e] = __popc(peers);
    __syncthreads();
    // exclusive scan over warps, one thread per expert
    for (int x = tid; x < num_experts; x += ALIGN_THREADS) {
      int acc = running[x];
      for (int w = 0; w < ALIGN_WARPS; ++w) {
        const int c = warp_cnt[w * num_experts + x];
        warp_cnt[w * num_experts + x] = acc;
        acc += c;
      }
      running[x] = acc;
    }
    __syncthreads();
    if (e >= 0) {
      const int pos = seg_off[e] + warp_cnt[warp * num_experts + e] + rank_in_warp;
      if (pos < sorted_capacity) sorted_token_ids[pos] = slot;
    }
    __syncthreads();
  }
}

// dst[p, :] = src[sorted_token_ids[p] / top_k, :]  (zeros for sentinel rows).
// 16-byte vectors; one warp per row chunk keeps the accesses coalesced.
__global__ void __launch_bounds__(256) moe_permute_rows_kernel(const uint4* __restrict__ src,
                                                               uint4* __restrict__ dst,
                                                               const int32_t* __restrict__ sorted_token_ids,
                                                               const int32_t* __restrict__ num_post_padded,
                                                               int numel, int top_k, int row_vecs,
                                                               int64_t src_row_vecs, int sorted_capacity) {
  const int rows = min(num_post_padded[0], sorted_capacity);
  for (int p = blockIdx.x; p < rows; p += gridDim.x) {
    const int sid = sorted_token_ids[p];
    uint4* d = dst + (int64_t)p * row_vecs;
    if (sid < numel) {
      const uint4* s = src + (int64_t)(sid / top_k) * src_row_vecs;
      for (int v = threadIdx.x; v < row_vecs; v += blockDim.x) d[v] = __ldg(s + v);
    } else {
      for (int v = threadIdx.x; v < row_vecs; v += blockDim.x) d[v] = make_uint4(0, 0, 0, 0);
    }
  }
}

// out[t, :] = sum_k partial[t * top_k + k, :]  accumulated in fp32, rounded once
// (torch's bf16 `sum(dim=1)`, python/dlBLAS/dlblas/kernels/fused_moe.py:375).
// With `topk_ids` given, a slot whose id lies outside [id_lo, id_hi) adds nothing: no kernel wrote its row
// (the reference zero-fills the whole buffer for that case, fused_moe.py:329-332,355-358).
template <typename T>
__global__ void __launch_bounds__(256) moe_combine_kernel(const T* __restrict__ partial, T* __restrict__ out,
                                                          int64_t tokens, int top_k, int hidden,
                                                          int64_t out_row_stride, const void* __restrict__ topk_ids,
                                                          int ids_are_int64, int64_t id_lo, int64_t id_hi) {
  using T2 = typename Elem<T>::T2;
  const int vecs = hidden / 8;
  const int64_t total = tokens * (int64_t)vecs;
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / vecs;
    const int v = (int)(idx - t * vecs);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int k = 0; k < top_k; ++k) {
      // the row is fetched whether or not its slot counts (every slot has a row in the buffer), so that the
      // row's load does not wait for the id's; a slot that does not count is dropped after the fact
      uint4 x = __ldcs(reinterpret_cast<const uint4*>(partial + (t * top_k + k) * (int64_t)hidden) + v);
      if (topk_ids != nullptr) {
        const int64_t id = ids_are_int64 ? __ldg(reinterpret_cast<const int64_t*>(topk_ids) + t * top_k + k)
                                         : (int64_t)__ldg(reinterpret_cast<const int32_t*>(topk_ids) + t * top_k + k);
        if (id < id_lo || id >= id_hi) x = make_uint4(0u, 0u, 0u, 0u);
      }
      const T2* x2 = reinterpret_cast<const T2*>(&x);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = Elem<T>::to_f2(x2[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    }
    uint4 o;
    T2* o2 = reinterpret_cast<T2*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) o2[j] = Elem<T>::from_f2(acc[2 * j], acc[2 * j + 1]);
    *(reinterpret_cast<uint4*>(out + t * out_row_stride) + v) = o;
  }
}

// Per-expert [start, end) ranges inside the ascending sort of the flattened ids
// (python/dlBLAS/dlblas/kernels/fused_moe.py:238-293): start = number of ids smaller than the expert's
// (negative ids sort first and count), end = start + the expert's count; an expert without slots gets
// start = end = 0, as the reference's kernel leaves it.  One CTA; counts are integer adds, so the result
// does not depend on the order of the atomics.
template <typename IdT, typename OutT>
__global__ void __launch_bounds__(ALIGN_THREADS) moe_start_end_kernel(const IdT* __restrict__ topk_ids, int numel,
                                                                      int num_experts, OutT* __restrict__ exp_start,
                                                                      OutT* __restrict__ exp_end) {
  extern __shared__ int32_t smem[];
  int32_t* counts = smem;            // [E + 1]; entry E counts the negative ids
  const int tid = threadIdx.x;
  for (int e = tid; e <= num_experts; e += ALIGN_THREADS) counts[e] = 0;
  __syncthreads();
  for (int i = tid; i < numel; i += ALIGN_THREADS) {
    const int64_t e = (int64_t)topk_ids[i];
    if (e < 0) atomicAdd(&counts[num_experts], 1);
    else if (e < num_experts) atomicAdd(&counts[(int)e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int acc = counts[num_experts];
    for (int e = 0; e < num_experts; ++e) {
      const int c = counts[e];
      exp_start[e] = (OutT)(c > 0 ? acc : 0);
      exp_end[e] = (OutT)(c > 0 ? acc + c : 0);
      acc += c;
    }
  }
}

}  // namespace dlb

extern "C" int dlb_moe_start_end(const void* topk_ids, int ids_are_int64, int64_t numel, int num_experts,
                                 void* exp_start, void* exp_end, int out_is_int64, void* stream) {
  DLB_NVTX("dlb_moe_start_end");
  using namespace dlb;
  DLB_CHECK_ARG(numel >= 0 && numel < (1LL << 30), DLB_ERR_TOO_LARGE, "moe_start_end: numel=%lld out of range",
                (long long)numel);
  DLB_CHECK_ARG(num_experts >= 1 && num_experts <= 1024, DLB_ERR_UNSUPPORTED,
                "moe_start_end: experts=%d not in [1,1024]", num_experts);
  DLB_CHECK_ARG(exp_start && exp_end && (numel == 0 || topk_ids), DLB_ERR_BAD_ARG, "moe_start_end: null pointer");
  const size_t smem = sizeof(int32_t) * ((size_t)num_experts + 1);
  cudaStream_t s = (cudaStream_t)stream;
  const int n = (int)numel;
  if (ids_are_int64 && out_is_int64)
    moe_start_end_kernel<int64_t, int64_t><<<1, ALIGN_THREADS, smem, s>>>((const int64_t*)topk_ids, n, num_experts,
                                                                         (int64_t*)exp_start, (int64_t*)exp_end);
  else if (ids_are_int64)
    moe_start_end_kernel<int64_t, int32_t><<<1, ALIGN_THREADS, smem, s>>>((const int64_t*)topk_ids, n, num_experts,
                                                                         (int32_t*)exp_start, (int32_t*)exp_end);
  else if (out_is_int64)
    moe_start_end_kernel<int32_t, int64_t><<<1, ALIGN_THREADS, smem, s>>>((const int32_t*)topk_ids, n, num_experts,
                                                                         (int64_t*)exp_start, (int64_t*)exp_end);
  else
    moe_start_end_kernel<int32_t, int32_t><<<1, ALIGN_THREADS, smem, s>>>((const int32_t*)topk_ids, n, num_experts,
                                                                         (int32_t*)exp_start, (int32_t*)exp_end);
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

extern "C" int dlb_moe_align_block_size(const void* topk_ids, int ids_are_int64, int64_t numel, int num_experts,
                                        int block, int32_t* sorted_token_ids, int64_t sorted_capacity,
                                        int32_t* expert_ids, int64_t expert_ids_capacity,
                                        int32_t* num_tokens_post_padded, int32_t* block_start, void* stream) {
  DLB_NVTX("dlb_moe_align_block_size");
  using namespace dlb;
  DLB_CHECK_ARG(numel >= 0 && numel < (1LL << 30), DLB_ERR_TOO_LARGE, "moe_align: numel=%lld out of range",
                (long long)numel);
  DLB_CHECK_ARG(num_experts >= 1 && num_experts <= 1024, DLB_ERR_UNSUPPORTED, "moe_align: experts=%d not in [1,1024]",
                num_experts);
  DLB_CHECK_ARG(block >= 1, DLB_ERR_BAD_ARG, "moe_align: block=%d", block);
  DLB_CHECK_ARG(sorted_token_ids && expert_ids && num_tokens_post_padded && block_start, DLB_ERR_BAD_ARG,
                "moe_align: null output pointer");
  DLB_CHECK_ARG(numel == 0 || topk_ids != nullptr, DLB_ERR_BAD_ARG, "moe_align: null topk_ids");
  // worst case padded length: every expert wastes block-1 entries
  const int64_t worst = numel + (int64_t)num_experts * (block - 1);
  const int64_t need = numel == 0 ? 0 : (worst < (numel + block - 1) / block * block ? worst : worst);
  DLB_CHECK_ARG(sorted_capacity >= need && sorted_capacity < (1LL << 31), DLB_ERR_BAD_ARG,
                "moe_align: sorted_token_ids capacity %lld < %lld", (long long)sorted_capacity, (long long)need);
  DLB_CHECK_ARG(expert_ids_capacity >= (need + block - 1) / block, DLB_ERR_BAD_ARG,
                "moe_align: expert_ids capacity %lld too small", (long long)expert_ids_capacity);
  const size_t smem = sizeof(int32_t) * ((size_t)num_experts * (3 + ALIGN_WARPS) + 1);
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e;
  if (ids_are_int64) {
    e = cudaFuncSetAttribute(moe_align_kernel<int64_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_last_error("moe_align: smem attribute: %s", cudaGetErrorString(e)); return (int)e; }
    moe_align_kernel<int64_t><<<1, ALIGN_THREADS, smem, s>>>(
        (const int64_t*)topk_ids, sorted_token_ids, expert_ids, num_tokens_post_padded, block_start, (int)numel,
        num_experts, block, (int)sorted_capacity, (int)expert_ids_capacity);
  } else {
    e = cudaFuncSetAttribute(moe_align_kernel<int32_t>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) { set_last_error("moe_align: smem attribute: %s", cudaGetErrorString(e)); return (int)e; }
    moe_align_kernel<int32_t><<<1, ALIGN_THREADS, smem, s>>>(
        (const int32_t*)topk_ids, sorted_token_ids, expert_ids, num_tokens_post_padded, block_start, (int)numel,
        num_experts, block, (int)sorted_capacity, (int)expert_ids_capacity);
  }
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

extern "C" int dlb_moe_permute_rows(const void* src, void* dst, const int32_t* sorted_token_ids,
                                    const int32_t* num_tokens_post_padded, int64_t numel, int top_k,
                                    int64_t hidden, int64_t src_row_stride, int64_t sorted_capacity,
                                    int elem_size, void* stream) {
  DLB_NVTX("dlb_moe_permute_rows");
  using namespace dlb;
  DLB_CHECK_ARG(elem_size == 2 || elem_size == 4, DLB_ERR_UNSUPPORTED, "moe_permute: element size %d", elem_size);
  DLB_CHECK_ARG(top_k >= 1 && numel >= 0 && hidden >= 0, DLB_ERR_BAD_ARG, "moe_permute: bad sizes");
  if (sorted_capacity == 0 || hidden == 0) return DLB_OK;
  const int64_t row_bytes = hidden * elem_size;
  DLB_CHECK_ARG(row_bytes % 16 == 0 && (src_row_stride * elem_size) % 16 == 0, DLB_ERR_ALIGNMENT,
                "moe_permute: rows must be multiples of 16 bytes");
  DLB_CHECK_ARG((((uintptr_t)src | (uintptr_t)dst) & 15) == 0, DLB_ERR_ALIGNMENT, "moe_permute: unaligned pointer");
  DLB_CHECK_ARG(sorted_capacity < (1LL << 31), DLB_ERR_TOO_LARGE, "moe_permute: capacity too large");
  int64_t blocks = sorted_capacity;
  const int64_t cap = (int64_t)sm_count(current_device()) * 16;
  if (blocks > cap) blocks = cap;
  moe_permute_rows_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(
      (const uint4*)src, (uint4*)dst, sorted_token_ids, num_tokens_post_padded, (int)numel, top_k,
      (int)(row_bytes / 16), src_row_stride * elem_size / 16, (int)sorted_capacity);
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

extern "C" int dlb_moe_combine(const void* partial, void* out, int64_t tokens, int top_k, int64_t hidden,
                               int64_t out_row_stride, int dtype, const void* topk_ids, int ids_are_int64,
                               int64_t id_lo, int64_t id_hi, void* stream) {
  DLB_NVTX("dlb_moe_combine");
  using namespace dlb;
  DLB_CHECK_ARG(tokens >= 0 && top_k >= 1 && hidden >= 0, DLB_ERR_BAD_ARG, "moe_combine: bad sizes");
  if (tokens == 0 || hidden == 0) return DLB_OK;
  DLB_CHECK_ARG(hidden % 8 == 0 && out_row_stride % 8 == 0, DLB_ERR_ALIGNMENT,
                "moe_combine: hidden and row stride must be multiples of 8");
  DLB_CHECK_ARG((((uintptr_t)partial | (uintptr_t)out) & 15) == 0, DLB_ERR_ALIGNMENT, "moe_combine: unaligned pointer");
  const int64_t total = tokens * (hidden / 8);
  int64_t blocks = (total + 255) / 256;
  const int64_t cap = (int64_t)sm_count(current_device()) * 16;
  if (blocks > cap) blocks = cap;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DLB_DTYPE_BF16) {
    moe_combine_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>(
        (const __nv_bfloat16*)partial, (__nv_bfloat16*)out, tokens, top_k, (int)hidden, out_row_stride, topk_ids,
        ids_are_int64, id_lo, id_hi);
  } else if (dtype == DLB_DTYPE_F16) {
    moe_combine_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>((const __half*)partial, (__half*)out, tokens, top_k,
                                                                 (int)hidden, out_row_stride, topk_ids, ids_are_int64,
                                                                 id_lo, id_hi);
  } else {
    set_last_error("moe_combine: unsupported dtype %d", dtype);
    return DLB_ERR_UNSUPPORTED;
  }
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}
