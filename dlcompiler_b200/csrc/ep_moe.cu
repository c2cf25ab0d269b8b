// Expert-parallel token exchange over NVLink peer memory (one process per GPU).
//
// The reference has no collective code at all; its expert-parallel hook leaves
// tokens replicated (python/dlBLAS/dlblas/kernels/fused_moe.py:113-114, 329-332).
// Here tokens are sharded: every rank sorts its (token, k) slots by expert, the
// ranks exchange their per-expert counts, and each rank then stores its rows
// DIRECTLY into the destination rank's receive buffer with plain peer stores,
// already in the expert-major, 128-row-block-padded layout the grouped GEMM
// consumes.  No host round trip, no staging copy, no library collective: the
// whole step is a fixed sequence of kernel launches.
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
                                                  int* status, int site) {
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
        if (now - t0 > DLB_WAIT_BUDGET_NS) {
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

struct EpPlanParams {
  const int32_t* expert_prefix;   // [E + 1] prefix of this rank's per-expert slot counts (moe_align, block 1)
  PeerPtrs counts;                // counts_sym of every rank
  PeerPtrs flags;                 // flags_sym of every rank
  int32_t* dest_base;             // [E] out: first row, in the owner's rows_sym, of this rank's slots of expert e
  int32_t* block_start;           // [E/G + 1] out: first 128-row block of each LOCAL expert
  int32_t* num_post_padded;       // [1] out
  int32_t* row_map;               // [cap] out: p if row p holds a token, cap otherwise
  int rank, world, experts, cap, epoch;
  int* status;
};

__global__ void __launch_bounds__(ep::PLAN_THREADS) ep_plan_kernel(const EpPlanParams p) {
  __shared__ int tot[ep::MAX_EXPERTS];      // rows of expert e over all ranks
  __shared__ int before[ep::MAX_EXPERTS];   // rows of expert e from ranks below mine
  __shared__ int lstart[ep::MAX_EXPERTS];   // local experts: first row / row count
  __shared__ int lcount[ep::MAX_EXPERTS];
  __shared__ int n_post;
  const int t = threadIdx.x;
  const int epr = p.experts / p.world;

  // 1. publish my counts into every rank's matrix (peer stores)
  for (int e = t; e < p.experts; e += ep::PLAN_THREADS) {
    const int c = p.expert_prefix[e + 1] - p.expert_prefix[e];
    for (int r = 0; r < p.world; ++r) reinterpret_cast<int32_t*>(p.counts.p[r])[p.rank * p.experts + e] = c;
  }
  __threadfence_system();
  __syncthreads();
  // 2. barrier: after it my own matrix is complete
  cross_gpu_barrier(p.flags, 0, p.rank, p.world, p.epoch, p.status, 41);
  __syncthreads();
  const volatile int32_t* cm = reinterpret_cast<const volatile int32_t*>(p.counts.p[p.rank]);
  for (int e = t; e < p.experts; e += ep::PLAN_THREADS) {
    int sum = 0, bef = 0;
    for (int s = 0; s < p.world; ++s) {
      const int c = cm[s * p.experts + e];
      if (s < p.rank) bef += c;
      sum += c;
    }
    tot[e] = sum;
    before[e] = bef;
  }
  __syncthreads();
  // 3. padded layouts of every rank's receive buffer (serial over experts, E <= 1024)
  if (t == 0) {
    for (int r = 0; r < p.world; ++r) {
      int acc = 0;
      for (int el = 0; el < epr; ++el) {
        const int e = r * epr + el;
        p.dest_base[e] = acc + before[e];
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
  // 4. which rows of my receive buffer will hold tokens
  for (int row = t; row < p.cap; row += ep::PLAN_THREADS) {
    int v = p.cap;
    if (row < n_post) {
      int el = 0;
      while (el + 1 < epr && lstart[el + 1] <= row) ++el;
      if (row - lstart[el] < lcount[el]) v = row;
    }
    p.row_map[row] = v;
  }
}

struct EpDispatchParams {
  const void* hidden;             // [T, H] this rank's tokens
  const void* topk_ids;           // [T * top_k] GLOBAL expert ids (int32 or int64)
  const float* topk_weights;      // [T * top_k]
  const int32_t* sorted_slots;    // [numel] slots sorted by expert
  const int32_t* expert_prefix;   // [E + 1]
  const int32_t* dest_base;       // [E]
  PeerPtrs rows, w, meta;         // rows_sym / w_sym / meta_sym of every rank
  int64_t hidden_row_stride;      // elements
  int numel, top_k, row_vecs /* H * elemsize / 16 */, experts, world, rank, cap, ids_are_int64;
};

__global__ void __launch_bounds__(256) ep_dispatch_kernel(const EpDispatchParams p) {
  const int epr = p.experts / p.world;
  for (int j = blockIdx.x; j < p.numel; j += gridDim.x) {
    const int slot = p.sorted_slots[j];
    if (slot < 0 || slot >= p.numel) continue;   // slots whose id was out of range are absent from the list
    const int e = p.ids_are_int64 ? (int)reinterpret_cast<const int64_t*>(p.topk_ids)[slot]
                                  : reinterpret_cast<const int32_t*>(p.topk_ids)[slot];
    if (e < 0 || e >= p.experts) continue;
    const int r = e / epr;
    const int pos = p.dest_base[e] + (j - p.expert_prefix[e]);
    if (pos >= p.cap) continue;
    const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const uint8_t*>(p.hidden) +
                                                      (int64_t)(slot / p.top_k) * p.hidden_row_stride * 2);
    uint4* dst = reinterpret_cast<uint4*>(p.rows.p[r]) + (int64_t)pos * p.row_vecs;
    for (int v = threadIdx.x; v < p.row_vecs; v += blockDim.x) dst[v] = __ldg(src + v);
    if (threadIdx.x == 0) {
      reinterpret_cast<float*>(p.w.p[r])[pos] = p.topk_weights[slot];
      reinterpret_cast<int32_t*>(p.meta.p[r])[pos] = (p.rank << 24) | slot;
    }
  }
  __threadfence_system();   // peer stores are performed before the barrier kernel that follows signals
}

__global__ void __launch_bounds__(32) ep_barrier_kernel(const PeerPtrs flags, int slot, int rank, int world,
                                                        int epoch, int* status) {
  cross_gpu_barrier(flags, slot, rank, world, epoch, status, 42 + slot);
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

extern "C" int dlb_ep_plan(const int32_t* expert_prefix, void* const* counts_sym, void* const* flags_sym,
                           int32_t* dest_base, int32_t* block_start, int32_t* num_post_padded, int32_t* row_map,
                           int rank, int world, int experts, int64_t cap, int epoch, int32_t* status,
                           void* stream) {
  using namespace dlb;
  DLB_CHECK_ARG(world >= 1 && world <= ep::MAX_RANKS && rank >= 0 && rank < world, DLB_ERR_BAD_ARG,
                "ep_plan: rank %d of %d", rank, world);
  DLB_CHECK_ARG(experts >= world && experts <= ep::MAX_EXPERTS && experts % world == 0, DLB_ERR_BAD_ARG,
                "ep_plan: %d experts over %d ranks", experts, world);
  DLB_CHECK_ARG(cap >= 128 && cap % 128 == 0 && cap < (1LL << 24), DLB_ERR_BAD_ARG,
                "ep_plan: capacity %lld must be a multiple of 128 below 2^24", (long long)cap);
  DLB_CHECK_ARG(expert_prefix && dest_base && block_start && num_post_padded && row_map, DLB_ERR_BAD_ARG,
                "ep_plan: null pointer");
  EpPlanParams p;
  int rc = fill_ptrs(&p.counts, counts_sym, world, "counts");
  if (rc != DLB_OK) return rc;
  rc = fill_ptrs(&p.flags, flags_sym, world, "flags");
  if (rc != DLB_OK) return rc;
  p.expert_prefix = expert_prefix;
  p.dest_base = dest_base;
  p.block_start = block_start;
  p.num_post_padded = num_post_padded;
  p.row_map = row_map;
  p.rank = rank;
  p.world = world;
  p.experts = experts;
  p.cap = (int)cap;
  p.epoch = epoch;
  p.status = status;
  ep_plan_kernel<<<1, ep::PLAN_THREADS, 0, (cudaStream_t)stream>>>(p);
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

extern "C" int dlb_ep_dispatch(const void* hidden, int64_t hidden_row_stride, int64_t hidden_cols, int elem_size,
                               const void* topk_ids, int ids_are_int64, const float* topk_weights,
                               const int32_t* sorted_slots, const int32_t* expert_prefix, const int32_t* dest_base,
                               void* const* rows_sym, void* const* w_sym, void* const* meta_sym, int64_t numel,
                               int top_k, int rank, int world, int experts, int64_t cap, void* stream) {
  using namespace dlb;
  DLB_CHECK_ARG(world >= 1 && world <= ep::MAX_RANKS && rank >= 0 && rank < world, DLB_ERR_BAD_ARG,
                "ep_dispatch: rank %d of %d", rank, world);
  DLB_CHECK_ARG(elem_size == 2, DLB_ERR_UNSUPPORTED, "ep_dispatch: 16-bit rows only");
  DLB_CHECK_ARG((hidden_cols * elem_size) % 16 == 0 && (hidden_row_stride * elem_size) % 16 == 0 &&
                    (((uintptr_t)hidden) & 15) == 0,
                DLB_ERR_ALIGNMENT, "ep_dispatch: rows must be 16-byte aligned multiples of 16 bytes");
  DLB_CHECK_ARG(numel >= 0 && numel < (1LL << 24) && top_k >= 1, DLB_ERR_BAD_ARG, "ep_dispatch: bad sizes");
  if (numel == 0) return DLB_OK;
  DLB_CHECK_ARG(hidden && topk_ids && topk_weights && sorted_slots && expert_prefix && dest_base, DLB_ERR_BAD_ARG,
                "ep_dispatch: null pointer");
  EpDispatchParams p;
  int rc = fill_ptrs(&p.rows, rows_sym, world, "rows");
  if (rc != DLB_OK) return rc;
  rc = fill_ptrs(&p.w, w_sym, world, "weights");
  if (rc != DLB_OK) return rc;
  rc = fill_ptrs(&p.meta, meta_sym, world, "meta");
  if (rc != DLB_OK) return rc;
  p.hidden = hidden;
  p.topk_ids = topk_ids;
  p.topk_weights = topk_weights;
  p.sorted_slots = sorted_slots;
  p.expert_prefix = expert_prefix;
  p.dest_base = dest_base;
  p.hidden_row_stride = hidden_row_stride;
  p.numel = (int)numel;
  p.top_k = top_k;
  p.row_vecs = (int)(hidden_cols * elem_size / 16);
  p.experts = experts;
  p.world = world;
  p.rank = rank;
  p.cap = (int)cap;
  p.ids_are_int64 = ids_are_int64;
  int64_t blocks = numel;
  const int64_t limit = (int64_t)sm_count(current_device()) * 16;
  if (blocks > limit) blocks = limit;
  ep_dispatch_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(p);
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

extern "C" int dlb_ep_barrier(void* const* flags_sym, int slot, int rank, int world, int epoch, int32_t* status,
                              void* stream) {
  using namespace dlb;
  DLB_CHECK_ARG(world >= 1 && world <= ep::MAX_RANKS && rank >= 0 && rank < world, DLB_ERR_BAD_ARG,
                "ep_barrier: rank %d of %d", rank, world);
  DLB_CHECK_ARG(slot >= 0 && slot < 8, DLB_ERR_BAD_ARG, "ep_barrier: slot %d", slot);
  PeerPtrs f;
  const int rc = fill_ptrs(&f, flags_sym, world, "flags");
  if (rc != DLB_OK) return rc;
  ep_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(f, slot, rank, world, epoch, status);
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}
