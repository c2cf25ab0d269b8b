// Grouped (per-expert) GEMM for fused_moe on the 5th-generation tensor cores.
//
// Computes, for every 128-row block b of the expert-sorted, block-padded row
// list produced by moe_align_block_size,
//     C[rows of b, :] = A[rows of b, :] @ B[expert_ids[b]]^T        (fp32 accumulate)
// which is what the reference's Triton `fused_moe_kernel` does per expert
// (python/dlBLAS/dlblas/kernels/fused_moe.py:77-175; B is [E, N, K] with K
// contiguous).  Two epilogues cover the two GEMMs of fused_moe():
//   FUSE_SILU   : B holds [gate; up] halves (fused_moe.py:351-352).  A tile
//                 accumulates 128 gate and the matching 128 up columns in one
//                 256-wide MMA and stores silu(gate) * up, rounding at the
//                 same three points as the reference (GEMM output -> bf16,
//                 silu -> bf16, product -> bf16).
//   WEIGHT/SCATTER: rows are scaled by the routing weight in fp32 before the
//                 cast (fused_moe.py:162-166) and written to row `slot` of the
//                 [tokens * top_k, N] buffer (reindex_c, fused_moe.py:168-169).
//
// Kernel structure (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: 128B-swizzled A (128 x 64) and B (256 x 64)
//               tiles into a 4-stage shared-memory ring, mbarrier expect_tx
//   warp 1      allocates TMEM, one lane issues tcgen05.mma (M128 N256 K16),
//               tcgen05.commit releases ring stages and publishes accumulators
//   warps 2-5   epilogue: tcgen05.ld of the fp32 accumulator (one TMEM lane =
//               one output row per thread), fused math, 16-byte global stores
// The 512 TMEM columns hold two 256-column accumulators, so the epilogue of
// tile i overlaps the main loop of tile i+1.  Tiles are ordered expert-major,
// then by N tile, then by M block, so the CTAs running concurrently share one
// expert's weight tiles through L2 and each weight tile leaves HBM once.
#include "common.cuh"

namespace dlb {

namespace gg {
constexpr int BM = 128;
constexpr int BK = 64;            // 64 x 16-bit = one 128-byte swizzle row
constexpr int UMMA_N = 256;
constexpr int UMMA_K = 16;
constexpr int STAGES = 4;
// (An explicit TMA L2 prefetch of the weight tiles 6 k-blocks ahead of the ring's loads was measured on
// B200 at the benchmark shape and made the step 18 % SLOWER: the 8 CTAs that share a weight tile all
// prefetch it, and the extra TMA traffic competes with the loads.  It is not in the code.)
constexpr int A_BYTES = BM * BK * 2;        // 16 KiB
constexpr int B_BYTES = UMMA_N * BK * 2;    // 32 KiB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int MAX_EXPERTS = 1024;
constexpr int THREADS = 192;
constexpr int TMEM_COLS = 512;
// dynamic shared memory: ring + 1 KiB alignment slack + control block
constexpr int CTRL_BYTES = 256 + (MAX_EXPERTS + 1) * 4;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + CTRL_BYTES;

constexpr int FLAG_FUSE_SILU = 1;
constexpr int FLAG_WEIGHT = 2;
constexpr int FLAG_SCATTER = 4;
constexpr int FLAG_PEER = 8;       // scatter to (rank, slot) taken from row_meta: plain stores into peer memory
constexpr int MAX_PEERS = 16;
}  // namespace gg

struct GroupedGemmParams {
  const int32_t* sorted_token_ids;   // [padded rows]
  const int32_t* block_start;        // [E + 1] first 128-row block of each expert
  const float* topk_weights;         // [numel] routing weight per slot (FLAG_WEIGHT)
  void* out;
  int64_t out_row_stride;            // elements
  int num_experts;
  int n_out;                         // output columns
  int k;                             // reduction length
  int numel;                         // tokens * top_k (sentinel value of sorted_token_ids)
  int rows_per_expert;               // rows of B per expert
  int up_row_offset;                 // FUSE_SILU: row offset of the `up` half inside an expert
  int max_m_blocks;                  // rows of A / 128
  int idesc;
  int* status;
  const int32_t* row_meta;           // FLAG_PEER: (source rank << 24) | slot for every row
  void* peer_out[gg::MAX_PEERS];     // FLAG_PEER: base of every rank's result buffer
  // optional cross-GPU synchronisation (expert parallelism); null pointers switch it off
  const int* wait_flags;             // before the first load: wait until wait_flags[r] >= sync_epoch for r < sync_world
  int* signal_flags[gg::MAX_PEERS];  // after the last store: the last CTA writes sync_epoch to signal_flags[r][0]
  int* done_counter;                 // device counter used to find the last CTA (left at zero)
  int sync_world, sync_epoch;
  uint64_t wait_budget_ns;           // wall-clock limit of the wait on wait_flags
};

template <typename T> __device__ __forceinline__ uint32_t pack2(float a, float b);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <typename T> __device__ __forceinline__ float round_to(float a) { return Elem<T>::to_f(Elem<T>::from_f(a)); }

// silu(gate) * up with the reference's rounding points.
template <typename T> __device__ __forceinline__ float silu_mul_rounded(float gate_acc, float up_acc) {
  const float g = round_to<T>(gate_acc);
  const float u = round_to<T>(up_acc);
  const float s = round_to<T>(g / (1.0f + __expf(-g)));
  return s * u;  // rounded by the caller's pack
}

struct TileCursor {
  int e = 0;
  // maps a linear tile index to (expert, n tile, m block); tiles must be visited in increasing order
  __device__ __forceinline__ void locate(const int32_t* bs, int num_experts, int n_tiles, int tile, int& m_blk,
                                         int& n_blk) {
    while (e + 1 < num_experts && tile >= bs[e + 1] * n_tiles) ++e;
    const int first = bs[e];
    const int mb = bs[e + 1] - first;
    const int local = tile - first * n_tiles;
    n_blk = local / mb;
    m_blk = first + (local - n_blk * mb);
  }
};

template <typename T, int FLAGS>
__global__ void __launch_bounds__(gg::THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const GroupedGemmParams p) {
  using namespace gg;
  constexpr bool kSilu = (FLAGS & FLAG_FUSE_SILU) != 0;
  constexpr bool kWeight = (FLAGS & FLAG_WEIGHT) != 0;
  constexpr bool kScatter = (FLAGS & FLAG_SCATTER) != 0;
  constexpr bool kPeer = (FLAGS & FLAG_PEER) != 0;
  constexpr int BN_OUT = kSilu ? 128 : 256;   // output columns per tile

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint8_t* ctrl = smem + STAGES * STAGE_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);            // [STAGES]
  uint64_t* empty_bar = full_bar + STAGES;                           // [STAGES]
  uint64_t* tmem_full_bar = empty_bar + STAGES;                      // [2]
  uint64_t* tmem_empty_bar = tmem_full_bar + 2;                      // [2]
  uint32_t* tmem_base_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_base_slot + 1);
  int32_t* bs = reinterpret_cast<int32_t*>(ctrl + 256);              // [E + 1]

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  for (int i = threadIdx.x; i <= p.num_experts; i += THREADS) {
    int v = p.block_start[i];
    bs[i] = v < p.max_m_blocks ? v : p.max_m_blocks;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tmem_full_bar[i], 1);
      mbar_init(&tmem_empty_bar[i], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == 0 && lane == 0) {
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_base_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_base_slot;

  const int n_tiles = (p.n_out + BN_OUT - 1) / BN_OUT;
  const int total_tiles = bs[p.num_experts] * n_tiles;
  const int k_blocks = (p.k + BK - 1) / BK;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      struct Walker {
        TileCursor cur;
        int tile, kb, m_blk, n_blk;
        bool valid;
      };
      auto start_walker = [&](Walker& w) {
        w.tile = blockIdx.x;
        w.kb = 0;
        w.valid = w.tile < total_tiles;
        if (w.valid) w.cur.locate(bs, p.num_experts, n_tiles, w.tile, w.m_blk, w.n_blk);
      };
      auto advance = [&](Walker& w) {
        if (++w.kb == k_blocks) {
          w.kb = 0;
          w.tile += gridDim.x;
          w.valid = w.tile < total_tiles;
          if (w.valid) w.cur.locate(bs, p.num_experts, n_tiles, w.tile, w.m_blk, w.n_blk);
        }
      };
      if (p.wait_flags != nullptr) {
        // rows of A are stored by other GPUs: do not read them before every rank has signalled
        uint64_t t0 = 0;
        for (int r = 0; r < p.sync_world; ++r) {
          for (uint32_t spin = 0;; ++spin) {
            int v;
            asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p.wait_flags + r) : "memory");
            if (v >= p.sync_epoch) break;
            if ((spin & 0x3f) == 0x3f) {
              const uint64_t now = globaltimer_ns();
              if (t0 == 0) t0 = now;
              if (now - t0 > p.wait_budget_ns) {
                if (p.status != nullptr && atomicCAS(p.status, DLB_DEV_OK, DLB_DEV_WAIT_TIMEOUT) == DLB_DEV_OK) {
                  p.status[1] = 5;
                  p.status[2] = (int)blockIdx.x;
                  p.status[3] = r;
                }
                break;   // proceed on stale data rather than hang; the status word reports it
              }
            }
          }
        }
        __threadfence_system();
      }
      Walker ld;
      start_walker(ld);
      uint32_t it = 0;
      while (ld.valid) {
        const int s = it % STAGES;
        const uint32_t ph = (it / STAGES) & 1;
        if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, 1, ld.tile)) break;
        uint8_t* a_dst = smem + s * STAGE_BYTES;
        uint8_t* b_dst = a_dst + A_BYTES;
        const int b_row = ld.cur.e * p.rows_per_expert + ld.n_blk * BN_OUT;
        mbar_arrive_expect_tx(&full_bar[s], STAGE_BYTES);
        tma_load_2d(a_dst, &tmap_a, &full_bar[s], ld.kb * BK, ld.m_blk * BM);
        if constexpr (kSilu) {
          tma_load_2d(b_dst, &tmap_b, &full_bar[s], ld.kb * BK, b_row);
          tma_load_2d(b_dst + B_BYTES / 2, &tmap_b, &full_bar[s], ld.kb * BK, b_row + p.up_row_offset);
        } else {
          tma_load_2d(b_dst, &tmap_b, &full_bar[s], ld.kb * BK, b_row);
        }
        advance(ld);
        ++it;
      }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      uint32_t it = 0;
      uint32_t tile_iter = 0;
      bool ok = true;
      const uint64_t desc0 = make_smem_desc(smem_u32(smem), 16, 1024, 2);   // stage 0, A operand
      const uint32_t desc_lo0 = (uint32_t)desc0, desc_hi = (uint32_t)(desc0 >> 32);
      for (int tile = blockIdx.x; ok && tile < total_tiles; tile += gridDim.x, ++tile_iter) {
        const uint32_t acc = tile_iter & 1;
        const uint32_t acc_ph = (tile_iter >> 1) & 1;
        if (!mbar_wait(&tmem_empty_bar[acc], acc_ph ^ 1, abort_flag, p.status, 2, tile)) { ok = false; break; }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * UMMA_N;
        for (int kb = 0; kb < k_blocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t ph = (it / STAGES) & 1;
          if (!mbar_wait(&full_bar[s], ph, abort_flag, p.status, 3, tile)) { ok = false; break; }
          tc_fence_after_sync();
          // descriptors: only the 14-bit address field (bytes >> 4) in the low word moves
          const uint32_t a_lo = desc_lo0 + (uint32_t)s * (STAGE_BYTES >> 4);
          const uint32_t b_lo = a_lo + (A_BYTES >> 4);
          if (kb == 0) umma_ss_lohi<0>(d_tmem, a_lo, desc_hi, b_lo, desc_hi, (uint32_t)p.idesc);
          else umma_ss_lohi<1>(d_tmem, a_lo, desc_hi, b_lo, desc_hi, (uint32_t)p.idesc);
#pragma unroll
          for (int kk = 1; kk < BK / UMMA_K; ++kk) {
            // advance 32 bytes (16 elements) along K inside the 128-byte swizzle row
            umma_ss_lohi<1>(d_tmem, a_lo + kk * 2, desc_hi, b_lo + kk * 2, desc_hi, (uint32_t)p.idesc);
          }
          umma_commit(&empty_bar[s]);   // stage reusable once these MMAs have read it
        }
        if (ok) umma_commit(&tmem_full_bar[acc]);
      }
    }
  } else {
    // ------------------------------ epilogue ------------------------------
    const int quad = warp & 3;                  // TMEM lane quadrant this warp may read
    const int row_in_tile = quad * 32 + lane;
    TileCursor cur;
    uint32_t tile_iter = 0;
    T* out = reinterpret_cast<T*>(p.out);
    for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, ++tile_iter) {
      int m_blk, n_blk;
      cur.locate(bs, p.num_experts, n_tiles, tile, m_blk, n_blk);
      const uint32_t acc = tile_iter & 1;
      const uint32_t acc_ph = (tile_iter >> 1) & 1;
      bool ok = mbar_wait(&tmem_full_bar[acc], acc_ph, abort_flag, p.status, 4, tile);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * UMMA_N;
      const int sorted_row = m_blk * BM + row_in_tile;
      const int col0 = n_blk * BN_OUT;

      int64_t out_row = sorted_row;
      bool row_valid = true;
      float w = 1.0f;
      if constexpr (kWeight || kScatter || kPeer) {
        const int sid = p.sorted_token_ids[sorted_row];
        row_valid = sid < p.numel;
        if constexpr (kScatter) out_row = row_valid ? sid : 0;
        if constexpr (kWeight) w = row_valid ? p.topk_weights[sid] : 0.f;
      }
      T* orow = out + out_row * p.out_row_stride + col0;
      if constexpr (kPeer) {
        // the row goes back to the rank that sent it, at the slot it came from (peer memory, plain stores)
        const int meta = row_valid ? p.row_meta[sorted_row] : 0;
        orow = reinterpret_cast<T*>(p.peer_out[(meta >> 24) & (MAX_PEERS - 1)]) +
               (int64_t)(meta & 0xffffff) * p.out_row_stride + col0;
      }

      if constexpr (kSilu) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t g[32], u[32];
          tmem_ld_32x32b_x32(t_row + c * 32, g);
          tmem_ld_32x32b_x32(t_row + 128 + c * 32, u);
          tmem_wait_ld();
          uint32_t o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const float r0 = silu_mul_rounded<T>(__uint_as_float(g[2 * j]), __uint_as_float(u[2 * j]));
            const float r1 = silu_mul_rounded<T>(__uint_as_float(g[2 * j + 1]), __uint_as_float(u[2 * j + 1]));
            o[j] = pack2<T>(r0, r1);
          }
          if (row_valid) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = col0 + c * 32 + v * 8;
              if (col + 8 <= p.n_out)
                *reinterpret_cast<uint4*>(orow + c * 32 + v * 8) = make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
            }
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t a[32];
          tmem_ld_32x32b_x32(t_row + c * 32, a);
          tmem_wait_ld();
          uint32_t o[16];
#pragma unroll
          for (int j = 0; j < 16; ++j)
            o[j] = pack2<T>(__uint_as_float(a[2 * j]) * w, __uint_as_float(a[2 * j + 1]) * w);
          if (row_valid) {
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              const int col = col0 + c * 32 + v * 8;
              if (col + 8 <= p.n_out)
                *reinterpret_cast<uint4*>(orow + c * 32 + v * 8) = make_uint4(o[4 * v], o[4 * v + 1], o[4 * v + 2], o[4 * v + 3]);
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tmem_empty_bar[acc]);
    }
  }

  // ------------------------------ teardown ------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  if (p.done_counter != nullptr && threadIdx.x == 0) {
    // every thread's stores (into peer memory, or into local rows the peers will read) are ordered
    // before this thread by the barrier; one system-scope fence per CTA publishes them, and the CTA
    // that arrives last tells every rank that this GPU's rows are in place
    __threadfence_system();
    const int prev = atomicAdd(p.done_counter, 1);
    if (prev == (int)gridDim.x - 1) {
      *p.done_counter = 0;
      __threadfence_system();
      for (int r = 0; r < p.sync_world; ++r)
        asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p.signal_flags[r]), "r"(p.sync_epoch) : "memory");
    }
  }
}

template <typename T, int FLAGS>
static int launch_grouped(const CUtensorMap& ta, const CUtensorMap& tb, const GroupedGemmParams& p, int grid,
                          cudaStream_t stream) {
  auto kern = grouped_gemm_kernel<T, FLAGS>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, gg::SMEM_BYTES);
  if (e != cudaSuccess) {
    set_last_error("grouped_gemm: cannot raise dynamic shared memory to %d B: %s", gg::SMEM_BYTES,
                   cudaGetErrorString(e));
    return (int)e;
  }
  kern<<<grid, gg::THREADS, gg::SMEM_BYTES, stream>>>(ta, tb, p);
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

}  // namespace dlb

namespace dlb {
static int grouped_gemm_impl(const void* a, int64_t a_rows, int64_t a_row_stride, const void* b, int num_experts,
                             int64_t rows_per_expert, int64_t k, int64_t b_row_stride, void* out,
                             int64_t out_row_stride, int64_t n_out, const int32_t* sorted_token_ids,
                             const int32_t* block_start, const float* topk_weights, int64_t numel, int flags,
                             int dtype, int32_t* status, void* stream, const int32_t* row_meta,
                             void* const* peer_out, int num_peers, const int32_t* wait_flags = nullptr,
                             void* const* signal_flags = nullptr, int32_t* done_counter = nullptr,
                             int sync_world = 0, int sync_epoch = 0) {
  using namespace dlb::gg;
  DLB_CHECK_ARG(dtype == DLB_DTYPE_BF16 || dtype == DLB_DTYPE_F16, DLB_ERR_UNSUPPORTED,
                "grouped_gemm: dtype %d (need fp16 or bf16)", dtype);
  DLB_CHECK_ARG(a && b && sorted_token_ids && block_start, DLB_ERR_BAD_ARG, "grouped_gemm: null pointer");
  DLB_CHECK_ARG(out != nullptr || (flags & FLAG_PEER), DLB_ERR_BAD_ARG, "grouped_gemm: null output");
  DLB_CHECK_ARG(num_experts >= 1 && num_experts <= MAX_EXPERTS, DLB_ERR_UNSUPPORTED, "grouped_gemm: experts=%d",
                num_experts);
  DLB_CHECK_ARG(a_rows >= 0 && a_rows % BM == 0, DLB_ERR_BAD_ARG,
                "grouped_gemm: A must hold a whole number of 128-row blocks (rows=%lld)", (long long)a_rows);
  DLB_CHECK_ARG(k >= 8 && k % 8 == 0, DLB_ERR_ALIGNMENT, "grouped_gemm: K=%lld must be a positive multiple of 8",
                (long long)k);
  DLB_CHECK_ARG(n_out >= 8 && n_out % 8 == 0 && out_row_stride % 8 == 0, DLB_ERR_ALIGNMENT,
                "grouped_gemm: N=%lld and the output row stride must be multiples of 8", (long long)n_out);
  DLB_CHECK_ARG((((uintptr_t)out) & 15) == 0, DLB_ERR_ALIGNMENT, "grouped_gemm: output not 16-byte aligned");
  DLB_CHECK_ARG(a_row_stride >= k && b_row_stride >= k, DLB_ERR_BAD_ARG, "grouped_gemm: row stride < K");
  DLB_CHECK_ARG(k < (1LL << 31) && n_out < (1LL << 31) && a_rows < (1LL << 31) && numel < (1LL << 31) &&
                    (int64_t)num_experts * rows_per_expert < (1LL << 31),
                DLB_ERR_TOO_LARGE, "grouped_gemm: a dimension exceeds int32");
  const bool silu = (flags & FLAG_FUSE_SILU) != 0;
  if (silu) {
    DLB_CHECK_ARG(flags == FLAG_FUSE_SILU, DLB_ERR_UNSUPPORTED, "grouped_gemm: silu fusion excludes weight/scatter");
    DLB_CHECK_ARG(rows_per_expert == 2 * n_out, DLB_ERR_BAD_ARG,
                  "grouped_gemm: fused silu needs rows_per_expert == 2 * n_out");
  } else {
    DLB_CHECK_ARG(rows_per_expert >= n_out, DLB_ERR_BAD_ARG, "grouped_gemm: rows_per_expert < n_out");
    if (flags & FLAG_WEIGHT) DLB_CHECK_ARG(topk_weights != nullptr, DLB_ERR_BAD_ARG, "grouped_gemm: null weights");
  }
  if (flags & FLAG_PEER) {
    DLB_CHECK_ARG(row_meta != nullptr && peer_out != nullptr && num_peers >= 1 && num_peers <= MAX_PEERS,
                  DLB_ERR_BAD_ARG, "grouped_gemm: peer scatter needs row_meta and 1..%d peer buffers", MAX_PEERS);
    for (int i = 0; i < num_peers; ++i)
      DLB_CHECK_ARG(peer_out[i] != nullptr && (((uintptr_t)peer_out[i]) & 15) == 0, DLB_ERR_ALIGNMENT,
                    "grouped_gemm: peer buffer %d is null or unaligned", i);
  }
  if (a_rows == 0) return DLB_OK;

  CUtensorMap ta, tb;
  int rc = make_tmap_2d_16b(&ta, a, (uint64_t)k, (uint64_t)a_rows, (uint64_t)a_row_stride * 2, BK, BM);
  if (rc != DLB_OK) return rc;
  rc = make_tmap_2d_16b(&tb, b, (uint64_t)k, (uint64_t)num_experts * rows_per_expert, (uint64_t)b_row_stride * 2,
                        BK, silu ? 128 : 256);
  if (rc != DLB_OK) return rc;

  GroupedGemmParams p;
  p.sorted_token_ids = sorted_token_ids;
  p.block_start = block_start;
  p.topk_weights = topk_weights;
  p.out = out;
  p.out_row_stride = out_row_stride;
  p.num_experts = num_experts;
  p.n_out = (int)n_out;
  p.k = (int)k;
  p.numel = (int)numel;
  p.rows_per_expert = (int)rows_per_expert;
  p.up_row_offset = (int)n_out;
  p.max_m_blocks = (int)(a_rows / BM);
  p.idesc = (int)make_idesc_f16(BM, UMMA_N, dtype == DLB_DTYPE_BF16 ? 1u : 0u, 0u, 0u);
  p.status = status;
  p.row_meta = row_meta;
  for (int i = 0; i < MAX_PEERS; ++i) p.peer_out[i] = (peer_out != nullptr && i < num_peers) ? peer_out[i] : nullptr;
  DLB_CHECK_ARG(sync_world >= 0 && sync_world <= MAX_PEERS, DLB_ERR_BAD_ARG, "grouped_gemm: sync_world %d", sync_world);
  DLB_CHECK_ARG((signal_flags == nullptr) == (done_counter == nullptr), DLB_ERR_BAD_ARG,
                "grouped_gemm: signal flags and done counter go together");
  p.wait_flags = wait_flags;
  p.done_counter = done_counter;
  p.sync_world = sync_world;
  p.sync_epoch = sync_epoch;
  p.wait_budget_ns = wait_budget_ns();
  for (int i = 0; i < MAX_PEERS; ++i)
    p.signal_flags[i] = (signal_flags != nullptr && i < sync_world) ? (int*)signal_flags[i] : nullptr;
  if (signal_flags != nullptr)
    for (int i = 0; i < sync_world; ++i)
      DLB_CHECK_ARG(signal_flags[i] != nullptr, DLB_ERR_BAD_ARG, "grouped_gemm: null signal flag of rank %d", i);

  const int grid = sm_count(current_device());
  cudaStream_t s = (cudaStream_t)stream;
  const bool bf = dtype == DLB_DTYPE_BF16;
  switch (flags) {
    case FLAG_FUSE_SILU:
      return bf ? launch_grouped<__nv_bfloat16, FLAG_FUSE_SILU>(ta, tb, p, grid, s)
                : launch_grouped<__half, FLAG_FUSE_SILU>(ta, tb, p, grid, s);
    case 0:
      return bf ? launch_grouped<__nv_bfloat16, 0>(ta, tb, p, grid, s) : launch_grouped<__half, 0>(ta, tb, p, grid, s);
    case FLAG_WEIGHT:
      return bf ? launch_grouped<__nv_bfloat16, FLAG_WEIGHT>(ta, tb, p, grid, s)
                : launch_grouped<__half, FLAG_WEIGHT>(ta, tb, p, grid, s);
    case FLAG_SCATTER:
      return bf ? launch_grouped<__nv_bfloat16, FLAG_SCATTER>(ta, tb, p, grid, s)
                : launch_grouped<__half, FLAG_SCATTER>(ta, tb, p, grid, s);
    case FLAG_WEIGHT | FLAG_SCATTER:
      return bf ? launch_grouped<__nv_bfloat16, FLAG_WEIGHT | FLAG_SCATTER>(ta, tb, p, grid, s)
                : launch_grouped<__half, FLAG_WEIGHT | FLAG_SCATTER>(ta, tb, p, grid, s);
    case FLAG_WEIGHT | FLAG_PEER:
      return bf ? launch_grouped<__nv_bfloat16, FLAG_WEIGHT | FLAG_PEER>(ta, tb, p, grid, s)
                : launch_grouped<__half, FLAG_WEIGHT | FLAG_PEER>(ta, tb, p, grid, s);
    default:
      set_last_error("grouped_gemm: unsupported flag combination %d", flags);
      return DLB_ERR_UNSUPPORTED;
  }
}
}  // namespace dlb

extern "C" int dlb_moe_grouped_gemm(const void* a, int64_t a_rows, int64_t a_row_stride, const void* b,
                                    int num_experts, int64_t rows_per_expert, int64_t k, int64_t b_row_stride,
                                    void* out, int64_t out_row_stride, int64_t n_out,
                                    const int32_t* sorted_token_ids, const int32_t* block_start,
                                    const float* topk_weights, int64_t numel, int flags, int dtype,
                                    int32_t* status, void* stream) {
  DLB_NVTX("dlb_moe_grouped_gemm");
  DLB_CHECK_ARG((flags & dlb::gg::FLAG_PEER) == 0, DLB_ERR_BAD_ARG,
                "grouped_gemm: peer scatter is only available through dlb_moe_grouped_gemm_sync");
  return dlb::grouped_gemm_impl(a, a_rows, a_row_stride, b, num_experts, rows_per_expert, k, b_row_stride, out,
                                out_row_stride, n_out, sorted_token_ids, block_start, topk_weights, numel, flags,
                                dtype, status, stream, nullptr, nullptr, 0);
}

// Grouped GEMM with optional cross-GPU synchronisation for expert parallelism: waits, before its
// first load, until wait_flags[r] >= epoch for every rank r (A's rows are stored by other GPUs), and
// after its last store lets the last CTA write `epoch` to signal_flags[r] of every rank.
extern "C" int dlb_moe_grouped_gemm_sync(const void* a, int64_t a_rows, int64_t a_row_stride, const void* b,
                                         int num_experts, int64_t rows_per_expert, int64_t k, int64_t b_row_stride,
                                         void* out, void* const* peer_out, int num_peers, int64_t out_row_stride,
                                         int64_t n_out, const int32_t* sorted_token_ids,
                                         const int32_t* block_start, const float* row_weights,
                                         const int32_t* row_meta, int64_t numel, int flags, int dtype,
                                         const int32_t* wait_flags, void* const* signal_flags,
                                         int32_t* done_counter, int sync_world, int sync_epoch, int32_t* status,
                                         void* stream) {
  DLB_NVTX("dlb_moe_grouped_gemm_sync");
  using namespace dlb::gg;
  void* o = out;
  if ((flags & FLAG_PEER) && o == nullptr && peer_out != nullptr && num_peers > 0) o = peer_out[0];
  return dlb::grouped_gemm_impl(a, a_rows, a_row_stride, b, num_experts, rows_per_expert, k, b_row_stride, o,
                                out_row_stride, n_out, sorted_token_ids, block_start, row_weights, numel, flags,
                                dtype, status, stream, row_meta, peer_out, num_peers, wait_flags, signal_flags,
                                done_counter, sync_world, sync_epoch);
}
