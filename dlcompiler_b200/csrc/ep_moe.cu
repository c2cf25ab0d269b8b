// Expert-parallel token exchange over NVLink peer memory (one process per GPU).
//
// The reference has no collective code at all; its expert-parallel hook leaves
// tokens replicated (python/dlBLAS/dlblas/kernels/fused_moe.py:113-114, 329-332).
// Here tokens are sharded: every rank counts its (token, k) slots per expert, the
// ranks exchange the counts through peer stores, and each rank then stores its
// rows DIRECTLY into the destination rank's receive buffer, already in the
// expert-major, 128-row-block-padded layout the grouped GEMM consumes.  The
// grouped GEMMs wait on / raise the cross-GPU flags themselves, so a step is five
// launches (route, send, GEMM, GEMM, combine) with no host round trip, no staging
// copy and no library collective.
//
// Buffers with the suffix _sym are symmetric: every rank owns one of the same
// size and holds the device pointers of all peers' copies.
//   counts_sym  int32 [G][E]   row s = rank s's per-expert slot counts
//   flags_sym   int32 [slots][G] monotone epoch flags for the cross-GPU barriers
//   rows_sym    T     [cap][H] received rows (expert-major, block padded)
//   w_sym       f32   [cap]    routing weight of each received row
//   meta_sym    int32 [cap]    (source rank << 24) | source slot
// Cross-GPU waits are bounded: a rank that does not see its peers within the
// wall-clock budget records the fact in the status word and returns.
#include "common.cuh"

namespace dlb {

namespace ep {
constexpr int MAX_RANKS = 16;
constexpr int MAX_EXPERTS = 1024;
constexpr int PLAN_THREADS = 1024;
constexpr int FLAG_STRIDE = 16;   // flags of one barrier slot: FLAG_STRIDE ints, one per source rank
constexpr int SEND_THREADS = 512;
}  // namespace ep

struct PeerPtrs {
  void* p[ep::MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Signal every peer (slot, my rank) = epoch, then wait until every peer's flag in my own copy
// reached the epoch.  Executed by threads 0..world-1 of one CTA.  Returns false on timeout.
__device__ __forceinline__ bool cross_gpu_barrier(const PeerPtrs& flags, int slot, int rank, int world, int epoch,
                                                  int* status, int site, uint64_t budget_ns) {
  const int t = threadIdx.x;
  bool ok = true;
  if (t < world) {
    __threadfence_system();
    st_release_sys(reinterpret_cast<int*>(flags.p[t]) + slot * ep::FLAG_STRIDE + rank, epoch);
    const int* mine = reinterpret_cast<const int*>(flags.p[rank]) + slot * ep::FLAG_STRIDE + t;
    uint64_t t0 = 0;
    for (uint32_t it = 0;; ++it) {
      if (ld_acquire_sys(mine) >= epoch) break;
      if ((it & 0x3f) == 0x3f) {
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        if (now - t0 > budget_ns) {
          ok = false;
          if (status != nullptr && atomicCAS(status, DLB_DEV_OK, DLB_DEV_WAIT_TIMEOUT) == DLB_DEV_OK) {
            status[1] = site;
            status[2] = rank;
            status[3] = t;
          }
          break;
        }
      }
    }
    __threadfence_system();
  }
  return ok;
}

__global__ void __launch_bounds__(32) ep_barrier_kernel(const PeerPtrs flags, int slot, int rank, int world,
                                                        int epoch, int* status, uint64_t budget_ns) {
  cross_gpu_barrier(flags, slot, rank, world, epoch, status, 42 + slot, budget_ns);
}

// ----------------------------------------------------------------------------
// Fused routing step: histogram + count exchange + receive layout + per-slot destination rows.
// One CTA.  Replaces (moe_align with block 1) + ep_plan: the stable rank of every slot inside its
// expert is turned directly into the row it will occupy in the owner's receive buffer.
// ----------------------------------------------------------------------------
struct EpRouteParams {
  const void* topk_ids;           // [numel] GLOBAL expert ids
  PeerPtrs counts, flags;
  int32_t* dest_pos;              // [numel] out: row in the owner's rows_sym (-1: id out of range)
  int32_t* block_start;           // [E/G + 1]
  int32_t* num_post_padded;       // [1]
  int32_t* row_map;               // [cap]
  int numel, ids_are_int64, rank, world, experts, cap, epoch;
  int* status;
  uint64_t budget_ns;             // wall-clock limit of the cross-GPU wait
};

__device__ __forceinline__ int load_id(const void* ids, int i, int is64) {
  return is64 ? (int)reinterpret_cast<const int64_t*>(ids)[i] : reinterpret_cast<const int32_t*>(ids)[i];
}

__global__ void __launch_bounds__(ep::PLAN_THREADS) ep_route_kernel(const EpRouteParams p) {
  extern __shared__ int32_t sm[];
  const int E = p.experts;
  int32_t* counts = sm;                 // [E] my slots per expert
  int32_t* tot = counts + E;            // [E] rows per expert over all ranks
  int32_t* base = tot + E;              // [E] first destination row of my slots of expert e
  int32_t* running = base + E;          // [E] my slots of expert e placed so far
  int32_t* lstart = running + E;        // [E] local experts: first row
  int32_t* lcount = lstart + E;         // [E] local experts: rows
  int32_t* warp_cnt = lcount + E;       // [32][E]
  __shared__ int n_post;
  const int t = threadIdx.x, lane = t & 31, warp = t >> 5;
  const int epr = E / p.world;
  constexpr int NW = ep::PLAN_THREADS / 32;

  for (int e = t; e < E; e += ep::PLAN_THREADS) {
    counts[e] = 0;
    running[e] = 0;
  }
  __syncthreads();
  for (int i = t; i < p.numel; i += ep::PLAN_THREADS) {
    const int e = load_id(p.topk_ids, i, p.ids_are_int64);
    if (e >= 0 && e < E) atomicAdd(&counts[e], 1);
  }
  __syncthreads();
  for (int e = t; e < E; e += ep::PLAN_THREADS)
    for (int r = 0; r < p.world; ++r) reinterpret_cast<int32_t*>(p.counts.p[r])[p.rank * E + e] = counts[e];
  __threadfence_system();
  __syncthreads();
  cross_gpu_barrier(p.flags, 0, p.rank, p.world, p.epoch, p.status, 41, p.budget_ns);
  __syncthreads();
  const volatile int32_t* cm = reinterpret_cast<const volatile int32_t*>(p.counts.p[p.rank]);
  for (int e = t; e < E; e += ep::PLAN_THREADS) {
    int sum = 0, bef = 0;
    for (int s = 0; s < p.world; ++s) {
      const int c = cm[s * E + e];
      if (s < p.rank) bef += c;
      sum += c;
    }
    tot[e] = sum;
    base[e] = bef;                      // completed with the padded expert offset below
  }
  __syncthreads();
  if (t == 0) {
    for (int r = 0; r < p.world; ++r) {
      int acc = 0;
      for (int el = 0; el < epr; ++el) {
        const int e = r * epr + el;
        base[e] += acc;
        if (r == p.rank) {
          lstart[el] = acc;
          lcount[el] = tot[e];
          p.block_start[el] = acc / 128;
        }
        acc += (tot[e] + 127) / 128 * 128;
      }
      if (r == p.rank) {
        acc = min(acc, p.cap);
        p.block_start[epr] = acc / 128;
        p.num_post_padded[0] = acc;
        n_post = acc;
      }
    }
  }
  __syncthreads();
  for (int row = t; row < p.cap; row += ep::PLAN_THREADS) {
    int v = p.cap;
    if (row < n_post) {
      int el = 0;
      while (el + 1 < epr && lstart[el + 1] <= row) ++el;
      if (row - lstart[el] < lcount[el]) v = row;
    }
    p.row_map[row] = v;
  }
  // stable placement: slots in index order, PLAN_THREADS per round
  for (int first = 0; first < p.numel; first += ep::PLAN_THREADS) {
    for (int i = t; i < NW * E; i += ep::PLAN_THREADS) warp_cnt[i] = 0;
    __syncthreads();
    const int slot = first + t;
    int e = -1;
    if (slot < p.numel) {
      const int v = load_id(p.topk_ids, slot, p.ids_are_int64);
      if (v >= 0 && v < E) e = v;
    }
    const unsigned peers = __match_any_sync(0xffffffffu, e);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (e >= 0 && rank_in_warp == 0) warp_cnt[warp * E + e] = __popc(peers);
    __syncthreads();
    for (int x = t; x < E; x += ep::PLAN_THREADS) {
      int acc = running[x];
      for (int w = 0; w < NW; ++w) {
        const int c = warp_cnt[w * E + x];
        warp_cnt[w * E + x] = acc;
        acc += c;
      }
      running[x] = acc;
    }
    __syncthreads();
    if (slot < p.numel) p.dest_pos[slot] = e >= 0 ? base[e] + warp_cnt[warp * E + e] + rank_in_warp : -1;
    __syncthreads();
  }
}

// Slot-indexed dispatch; the last CTA to finish signals every rank (flag slot 1), nobody waits here.
struct EpSendParams {
  const void* hidden;
  const void* topk_ids;
  const float* topk_weights;
  const int32_t* dest_pos;
  PeerPtrs rows, w, meta, flags;
  int* done_counter;
  int64_t hidden_row_stride;
  int numel, top_k, row_vecs, experts, world, rank, cap, ids_are_int64, epoch;
};

// A few fat CTAs (two per SM) walk the slots, four rows in flight per pass, and each CTA issues ONE
// system-scope fence at its very end: the fence has to wait for every peer store the CTA still has on the
// links, so one CTA per slot (a fence per 8 KB row) cost 42 us for 1024 rows where the bytes need 10.
__global__ void __launch_bounds__(ep::SEND_THREADS) ep_send_kernel(const EpSendParams p) {
  const int epr = p.experts / p.world;
  constexpr int ROWS = 4;
  for (int first = blockIdx.x * ROWS; first < p.numel; first += gridDim.x * ROWS) {
    const uint4* src[ROWS];
    uint4* dst[ROWS];
#pragma unroll
    for (int j = 0; j < ROWS; ++j) {
      const int slot = first + j;
      src[j] = nullptr;
      dst[j] = nullptr;
      if (slot >= p.numel) continue;
      const int pos = p.dest_pos[slot];
      if (pos < 0 || pos >= p.cap) continue;
      const int r = load_id(p.topk_ids, slot, p.ids_are_int64) / epr;
      src[j] = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.hidden) +
                                              (int64_t)(slot / p.top_k) * p.hidden_row_stride * 2);
      dst[j] = reinterpret_cast<uint4*>(p.rows.p[r]) + (int64_t)pos * p.row_vecs;
      if (threadIdx.x == j) {
        reinterpret_cast<float*>(p.w.p[r])[pos] = p.topk_weights[slot];
        reinterpret_cast<int32_t*>(p.meta.p[r])[pos] = (p.rank << 24) | slot;
      }
    }
    for (int v = threadIdx.x; v < p.row_vecs; v += blockDim.x) {
      uint4 x[ROWS];
#pragma unroll
      for (int j = 0; j < ROWS; ++j)
        if (src[j] != nullptr) x[j] = __ldg(src[j] + v);
#pragma unroll
      for (int j = 0; j < ROWS; ++j)
        if (src[j] != nullptr) dst[j][v] = x[j];
    }
  }
  // one system-scope fence per CTA, after the barrier that orders every thread's peer stores before it
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const int prev = atomicAdd(p.done_counter, 1);
    if (prev == (int)gridDim.x - 1) {
      *p.done_counter = 0;
      __threadfence_system();
      for (int r = 0; r < p.world; ++r)
        st_release_sys(reinterpret_cast<int*>(p.flags.p[r]) + 1 * ep::FLAG_STRIDE + p.rank, p.epoch);
    }
  }
}

// Threads 0..world-1 of the CTA wait (bounded) until wait_flags[r] >= epoch, then the whole CTA proceeds.
__device__ __forceinline__ void wait_all_ranks(const int* wait_flags, int world, int epoch, int* status, int site,
                                               uint64_t budget_ns) {
  if (threadIdx.x < world) {
    uint64_t t0 = 0;
    for (uint32_t spin = 0;; ++spin) {
      if (ld_acquire_sys(wait_flags + threadIdx.x) >= epoch) break;
      if ((spin & 0x3f) == 0x3f) {
        const uint64_t now = globaltimer_ns();
        if (t0 == 0) t0 = now;
        if (now - t0 > budget_ns) {
          if (status != nullptr && atomicCAS(status, DLB_DEV_OK, DLB_DEV_WAIT_TIMEOUT) == DLB_DEV_OK) {
            status[1] = site;
            status[2] = (int)blockIdx.x;
            status[3] = (int)threadIdx.x;
          }
          break;
        }
      }
    }
    __threadfence_system();
  }
  __syncthreads();
}

// Top-k combine that first waits (bounded) until every rank has signalled flag slot 2.
template <typename T>
__global__ void __launch_bounds__(256) ep_combine_kernel(const T* __restrict__ partial, T* __restrict__ out,
                                                         int64_t tokens, int top_k, int hidden,
                                                         int64_t out_row_stride, const int* wait_flags, int world,
                                                         int epoch, int* status, const int32_t* __restrict__ dest_pos,
                                                         uint64_t budget_ns) {
  using T2 = typename Elem<T>::T2;
  wait_all_ranks(wait_flags, world, epoch, status, 44, budget_ns);
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
      // a slot that was sent nowhere (expert id out of range) has no row this step: its place in the
      // buffer still holds an earlier step's data
      if (dest_pos != nullptr && dest_pos[t * top_k + k] < 0) continue;
      // written by other GPUs during this step: bypass any stale cached copy
      const uint4 x = __ldcv(reinterpret_cast<const uint4*>(partial + (t * top_k + k) * (int64_t)hidden) + v);
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

// Top-k combine that PULLS: once every rank has signalled that its down projection is complete, each
// token's top-k rows are read straight out of the owners' result buffers (coalesced 16-byte peer loads
// over NVLink) and summed.  The expert side then writes its rows locally, in full cache lines, instead
// of pushing row fragments through the links from the GEMM epilogue.
struct EpPullParams {
  PeerPtrs y;                     // every rank's [cap][hidden] down-projection output
  const void* topk_ids;           // [tokens * top_k] GLOBAL expert ids
  const int32_t* dest_pos;        // [tokens * top_k] row inside the owner's buffer (from the route step)
  void* out;
  const int* wait_flags;
  int* status;
  int64_t y_row_stride, out_row_stride, tokens;
  int top_k, hidden, experts, world, cap, ids_are_int64, epoch;
  uint64_t budget_ns;
};

template <typename T>
__global__ void __launch_bounds__(256) ep_combine_pull_kernel(const EpPullParams p) {
  using T2 = typename Elem<T>::T2;
  wait_all_ranks(p.wait_flags, p.world, p.epoch, p.status, 45, p.budget_ns);
  const int vecs = p.hidden / 8;
  const int epr = p.experts / p.world;
  const int64_t total = p.tokens * (int64_t)vecs;
  T* out = reinterpret_cast<T*>(p.out);
  for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (int64_t)gridDim.x * blockDim.x) {
    const int64_t t = idx / vecs;
    const int v = (int)(idx - t * vecs);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    auto fetch = [&](int k) -> uint4 {
      const int slot = (int)(t * p.top_k + k);
      const int pos = p.dest_pos[slot];
      if (pos < 0 || pos >= p.cap) return make_uint4(0u, 0u, 0u, 0u);
      const int r = load_id(p.topk_ids, slot, p.ids_are_int64) / epr;
      // stored by another GPU during this step: never a cached copy
      return __ldcv(reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(p.y.p[r]) + (int64_t)pos * p.y_row_stride) + v);
    };
    auto add = [&](const uint4& x) {
      const T2* x2 = reinterpret_cast<const T2*>(&x);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = Elem<T>::to_f2(x2[j]);
        acc[2 * j] += f.x;
        acc[2 * j + 1] += f.y;
      }
    };
    int k = 0;
    for (; k + 2 <= p.top_k; k += 2) {   // two link round trips in flight per thread
      const uint4 x0 = fetch(k), x1 = fetch(k + 1);
      add(x0);
      add(x1);
    }
    if (k < p.top_k) add(fetch(k));
    uint4 o;
    T2* o2 = reinterpret_cast<T2*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) o2[j] = Elem<T>::from_f2(acc[2 * j], acc[2 * j + 1]);
    *(reinterpret_cast<uint4*>(out + t * p.out_row_stride) + v) = o;
  }
}

static int fill_ptrs(PeerPtrs* out, void* const* in, int world, const char* what) {
  DLB_CHECK_ARG(in != nullptr, DLB_ERR_BAD_ARG, "ep: null pointer table for %s", what);
  for (int i = 0; i < ep::MAX_RANKS; ++i) out->p[i] = nullptr;
  for (int i = 0; i < world; ++i) {
    DLB_CHECK_ARG(in[i] != nullptr && (((uintptr_t)in[i]) & 15) == 0, DLB_ERR_ALIGNMENT,
                  "ep: %s pointer of rank %d is null or not 16-byte aligned", what, i);
    out->p[i] = in[i];
  }
  return DLB_OK;
}

}  // namespace dlb

extern "C" int dlb_ep_barrier(void* const* flags_sym, int slot, int rank, int world, int epoch, int32_t* status,
                              void* stream) {
  DLB_NVTX("dlb_ep_barrier");
  using namespace dlb;
  DLB_CHECK_ARG(world >= 1 && world <= ep::MAX_RANKS && rank >= 0 && rank < world, DLB_ERR_BAD_ARG,
                "ep_barrier: rank %d of %d", rank, world);
  DLB_CHECK_ARG(slot >= 0 && slot < 8, DLB_ERR_BAD_ARG, "ep_barrier: slot %d", slot);
  PeerPtrs f;
  const int rc = fill_ptrs(&f, flags_sym, world, "flags");
  if (rc != DLB_OK) return rc;
  ep_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f, slot, rank, world, epoch, status, wait_budget_ns());
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

extern "C" int dlb_ep_route(const void* topk_ids, int ids_are_int64, int64_t numel, void* const* counts_sym,
                            void* const* flags_sym, int32_t* dest_pos, int32_t* block_start,
                            int32_t* num_post_padded, int32_t* row_map, int rank, int world, int experts,
                            int64_t cap, int epoch, int32_t* status, void* stream) {
  DLB_NVTX("dlb_ep_route");
  using namespace dlb;
  DLB_CHECK_ARG(world >= 1 && world <= ep::MAX_RANKS && rank >= 0 && rank < world, DLB_ERR_BAD_ARG,
                "ep_route: rank %d of %d", rank, world);
  DLB_CHECK_ARG(experts >= world && experts <= ep::MAX_EXPERTS && experts % world == 0, DLB_ERR_BAD_ARG,
                "ep_route: %d experts over %d ranks", experts, world);
  DLB_CHECK_ARG(cap >= 128 && cap % 128 == 0 && cap < (1LL << 24), DLB_ERR_BAD_ARG,
                "ep_route: capacity %lld must be a multiple of 128 below 2^24", (long long)cap);
  DLB_CHECK_ARG(numel >= 0 && numel < (1LL << 24), DLB_ERR_BAD_ARG, "ep_route: numel out of range");
  DLB_CHECK_ARG((numel == 0 || (topk_ids && dest_pos)) && block_start && num_post_padded && row_map,
                DLB_ERR_BAD_ARG, "ep_route: null pointer");
  EpRouteParams p;
  int rc = fill_ptrs(&p.counts, counts_sym, world, "counts");
  if (rc != DLB_OK) return rc;
  rc = fill_ptrs(&p.flags, flags_sym, world, "flags");
  if (rc != DLB_OK) return rc;
  p.topk_ids = topk_ids;
  p.dest_pos = dest_pos;
  p.block_start = block_start;
  p.num_post_padded = num_post_padded;
  p.row_map = row_map;
  p.numel = (int)numel;
  p.ids_are_int64 = ids_are_int64;
  p.rank = rank;
  p.world = world;
  p.experts = experts;
  p.cap = (int)cap;
  p.epoch = epoch;
  p.status = status;
  p.budget_ns = wait_budget_ns();
  const size_t smem = sizeof(int32_t) * (size_t)experts * (6 + ep::PLAN_THREADS / 32);
  cudaError_t e = cudaFuncSetAttribute(ep_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) {
    set_last_error("ep_route: smem attribute: %s", cudaGetErrorString(e));
    return (int)e;
  }
  ep_route_kernel<<<1, ep::PLAN_THREADS, smem, (cudaStream_t)stream>>>(p);
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

extern "C" int dlb_ep_send(const void* hidden, int64_t hidden_row_stride, int64_t hidden_cols, int elem_size,
                           const void* topk_ids, int ids_are_int64, const float* topk_weights,
                           const int32_t* dest_pos, void* const* rows_sym, void* const* w_sym,
                           void* const* meta_sym, void* const* flags_sym, int32_t* done_counter, int64_t numel,
                           int top_k, int rank, int world, int experts, int64_t cap, int epoch, void* stream) {
  DLB_NVTX("dlb_ep_send");
  using namespace dlb;
  DLB_CHECK_ARG(world >= 1 && world <= ep::MAX_RANKS && rank >= 0 && rank < world, DLB_ERR_BAD_ARG,
                "ep_send: rank %d of %d", rank, world);
  DLB_CHECK_ARG(elem_size == 2, DLB_ERR_UNSUPPORTED, "ep_send: 16-bit rows only");
  DLB_CHECK_ARG((hidden_cols * elem_size) % 16 == 0 && (hidden_row_stride * elem_size) % 16 == 0 &&
                    (((uintptr_t)hidden) & 15) == 0,
                DLB_ERR_ALIGNMENT, "ep_send: rows must be 16-byte aligned multiples of 16 bytes");
  DLB_CHECK_ARG(numel >= 0 && numel < (1LL << 24) && top_k >= 1 && done_counter != nullptr, DLB_ERR_BAD_ARG,
                "ep_send: bad sizes");
  DLB_CHECK_ARG(numel == 0 || (hidden && topk_ids && topk_weights && dest_pos), DLB_ERR_BAD_ARG,
                "ep_send: null pointer");
  EpSendParams p;
  int rc = fill_ptrs(&p.rows, rows_sym, world, "rows");
  if (rc != DLB_OK) return rc;
  rc = fill_ptrs(&p.w, w_sym, world, "weights");
  if (rc != DLB_OK) return rc;
  rc = fill_ptrs(&p.meta, meta_sym, world, "meta");
  if (rc != DLB_OK) return rc;
  rc = fill_ptrs(&p.flags, flags_sym, world, "flags");
  if (rc != DLB_OK) return rc;
  p.hidden = hidden;
  p.topk_ids = topk_ids;
  p.topk_weights = topk_weights;
  p.dest_pos = dest_pos;
  p.done_counter = done_counter;
  p.hidden_row_stride = hidden_row_stride;
  p.numel = (int)numel;
  p.top_k = top_k;
  p.row_vecs = (int)(hidden_cols * elem_size / 16);
  p.experts = experts;
  p.world = world;
  p.rank = rank;
  p.cap = (int)cap;
  p.ids_are_int64 = ids_are_int64;
  p.epoch = epoch;
  int64_t blocks = numel < 1 ? 1 : (numel + 3) / 4;
  const int64_t limit = (int64_t)sm_count(current_device()) * 2;
  if (blocks > limit) blocks = limit;
  ep_send_kernel<<<(unsigned)blocks, ep::SEND_THREADS, 0, (cudaStream_t)stream>>>(p);
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

extern "C" int dlb_ep_combine(const void* partial, void* out, int64_t tokens, int top_k, int64_t hidden,
                              int64_t out_row_stride, int dtype, const int32_t* wait_flags, int world, int epoch,
                              const int32_t* dest_pos, int32_t* status, void* stream) {
  DLB_NVTX("dlb_ep_combine");
  using namespace dlb;
  DLB_CHECK_ARG(tokens >= 0 && top_k >= 1 && hidden >= 0, DLB_ERR_BAD_ARG, "ep_combine: bad sizes");
  DLB_CHECK_ARG(world >= 1 && world <= ep::MAX_RANKS && wait_flags != nullptr, DLB_ERR_BAD_ARG,
                "ep_combine: bad wait arguments");
  DLB_CHECK_ARG(hidden % 8 == 0 && out_row_stride % 8 == 0, DLB_ERR_ALIGNMENT,
                "ep_combine: hidden and row stride must be multiples of 8");
  DLB_CHECK_ARG((((uintptr_t)partial | (uintptr_t)out) & 15) == 0, DLB_ERR_ALIGNMENT, "ep_combine: unaligned pointer");
  const int64_t total = tokens * (hidden / 8);
  int64_t blocks = (total + 255) / 256;
  if (blocks < 1) blocks = 1;   // the wait still has to happen so that the next step may reuse the buffers
  const int64_t limit = (int64_t)sm_count(current_device()) * 8;
  if (blocks > limit) blocks = limit;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DLB_DTYPE_BF16) {
    ep_combine_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>(
        (const __nv_bfloat16*)partial, (__nv_bfloat16*)out, tokens, top_k, (int)hidden, out_row_stride, wait_flags,
        world, epoch, status, dest_pos, wait_budget_ns());
  } else if (dtype == DLB_DTYPE_F16) {
    ep_combine_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>((const __half*)partial, (__half*)out, tokens, top_k,
                                                                (int)hidden, out_row_stride, wait_flags, world, epoch,
                                                                status, dest_pos, wait_budget_ns());
  } else {
    set_last_error("ep_combine: unsupported dtype %d", dtype);
    return DLB_ERR_UNSUPPORTED;
  }
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

extern "C" int dlb_ep_combine_pull(void* const* y_sym, int64_t y_row_stride, const void* topk_ids, int ids_are_int64,
                                   const int32_t* dest_pos, void* out, int64_t tokens, int top_k, int64_t hidden,
                                   int64_t out_row_stride, int dtype, const int32_t* wait_flags, int world,
                                   int experts, int64_t cap, int epoch, int32_t* status, void* stream) {
  DLB_NVTX("dlb_ep_combine_pull");
  using namespace dlb;
  DLB_CHECK_ARG(tokens >= 0 && top_k >= 1 && hidden >= 0 && tokens * top_k < (1LL << 24), DLB_ERR_BAD_ARG,
                "ep_combine_pull: bad sizes");
  DLB_CHECK_ARG(world >= 1 && world <= ep::MAX_RANKS && wait_flags != nullptr, DLB_ERR_BAD_ARG,
                "ep_combine_pull: bad wait arguments");
  DLB_CHECK_ARG(experts >= world && experts % world == 0, DLB_ERR_BAD_ARG, "ep_combine_pull: %d experts over %d ranks",
                experts, world);
  DLB_CHECK_ARG(hidden % 8 == 0 && out_row_stride % 8 == 0 && y_row_stride % 8 == 0, DLB_ERR_ALIGNMENT,
                "ep_combine_pull: hidden and row strides must be multiples of 8");
  DLB_CHECK_ARG((((uintptr_t)out) & 15) == 0, DLB_ERR_ALIGNMENT, "ep_combine_pull: unaligned output");
  DLB_CHECK_ARG(tokens == 0 || (topk_ids && dest_pos && out), DLB_ERR_BAD_ARG, "ep_combine_pull: null pointer");
  EpPullParams p;
  const int rc = fill_ptrs(&p.y, y_sym, world, "down-projection output");
  if (rc != DLB_OK) return rc;
  p.topk_ids = topk_ids;
  p.dest_pos = dest_pos;
  p.out = out;
  p.wait_flags = wait_flags;
  p.status = status;
  p.y_row_stride = y_row_stride;
  p.out_row_stride = out_row_stride;
  p.tokens = tokens;
  p.top_k = top_k;
  p.hidden = (int)hidden;
  p.experts = experts;
  p.world = world;
  p.cap = (int)cap;
  p.ids_are_int64 = ids_are_int64;
  p.epoch = epoch;
  p.budget_ns = wait_budget_ns();
  const int64_t total = tokens * (hidden / 8);
  int64_t blocks = (total + 255) / 256;
  if (blocks < 1) blocks = 1;   // the wait still has to happen so that the next step may reuse the buffers
  const int64_t limit = (int64_t)sm_count(current_device()) * 8;
  if (blocks > limit) blocks = limit;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DLB_DTYPE_BF16) {
    ep_combine_pull_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>(p);
  } else if (dtype == DLB_DTYPE_F16) {
    ep_combine_pull_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>(p);
  } else {
    set_last_error("ep_combine_pull: unsupported dtype %d", dtype);
    return DLB_ERR_UNSUPPORTED;
  }
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}
