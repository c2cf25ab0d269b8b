// Variable-length causal GQA flash-attention prefill on tcgen05 / TMEM.
//
// Math of the reference's context_attention_fwd
// (python/dlBLAS/dlblas/kernels/prefill_attention.py:28-181): per packed
// sequence, softmax(q k^T * sm_scale + causal mask) v with fp32 softmax and
// accumulation and P cast to the value dtype before P.V; optional LSE output
// in the convention of python/dlBLAS/dlblas/kernels/flash_attention.py:152-155
// (natural log, scale included).
//
// One CTA = one (sequence, q-head, 128-query tile); two CTAs are resident per
// SM (256 TMEM columns and ~97 KiB of shared memory each), so one CTA's
// softmax overlaps the other's MMAs.  Inside a CTA, 192 threads (moving registers to the softmax warps
// with setmaxnreg was tried: ptxas keeps allocating under the launch bound and spills):
//   warp 4     TMA producer: Q tile once, then K and V tiles of 64 keys into
//              2-stage rings (3-D tensor maps over [token, head, d], 128-byte swizzle; for a paged
//              cache 4-D maps over [page, slot, head, d] and one box per page of the block)
//   warp 5     one lane issues tcgen05.mma: S_j = Q K_j^T (M128 N64 K16 x 8) into
//              a double-buffered TMEM S, then O += P_{j-1} V_{j-1}
//              (M128 N128 K16 x 4, P as the A operand from TMEM, V as an MN-major operand
//              straight from the row-major tile), software-pipelined so S_j is computed while
//              the softmax of block j-1 runs; two commits per block (s_full also frees the K
//              stage, pv_done the V stage)
//   warps 0-3  softmax: one thread per query row reads its S row from TMEM
//              (tcgen05.ld), online softmax in the base-2 domain, writes P back with
//              tcgen05.st as 16-bit pairs over the first 32 columns of the same S buffer,
//              rescales O in TMEM only when the row max grew by more than
//              2^8 (lazy rescaling), and finally normalises and stores O
// CTAs are ordered (sequence, kv head) group by group, heavy causal tiles first inside a group, so the
// resident CTAs share K/V through L2 and the tail of each group is short.
//
// Built for tile widths D = 64 and 128.  Head sizes that are other multiples of 8 (and a v head size that
// differs from the q/k one, as the reference's paged kernel allows, paged_attention.py:526-539) run on the
// next width: the tensor maps carry the true sizes, so the copy engine zero-fills the missing columns of
// every Q, K and V tile in shared memory and nothing is copied or padded in global memory.
// V rows of the last key block that lie past the end of the keys are zeroed in shared memory before the
// P.V MMA reads them: their probabilities are exactly zero, but 0 x (stale NaN bits of a cache page) is NaN.
#include <math_constants.h>

#include <algorithm>

#include "common.cuh"

namespace dlb {

namespace fp {
constexpr int BM = 128;           // query rows per CTA
constexpr int BN = 64;            // keys per block
constexpr int THREADS = 192;      // warps 0-3 softmax (TMEM quadrant = warp id), warp 4 TMA, warp 5 MMA
constexpr int WARP_TMA = 4;
constexpr int WARP_MMA = 5;
constexpr int Q_BOX = BM * 128;   // one 64-wide (128 B) column box of the Q tile
constexpr int KV_BOX = BN * 128;  // one 64-wide column box of a K or V tile
constexpr int KV_STAGES = 2;
constexpr int TMEM_COLS = 256;    // S0 [0,64) S1 [64,128) O [128,128+D)
constexpr float RESCALE_THRESHOLD = 8.0f;   // log2 units
// (Computing a share of the exponentials with a degree-3 polynomial on the FMA pipe instead of the SFU,
// as large kernels of this kind do, was measured on B200 at 12.5 %, 25 % and 37.5 % of the scores and
// was 2 %, 4 % and 10 % slower on the 4 x 8192 benchmark: the softmax warps are bound by issue slots
// and latency, not by the SFU.  It is not in the code.)
// shared-memory layout for head size D (64 or 128)
template <int D> struct Layout {
  static constexpr int BOXES = D / 64;
  static constexpr int Q_BYTES = BOXES * Q_BOX;
  static constexpr int KV_BYTES = BOXES * KV_BOX;
  static constexpr int OFF_Q = 0;
  static constexpr int OFF_K = OFF_Q + Q_BYTES;
  static constexpr int OFF_V = OFF_K + KV_STAGES * KV_BYTES;
  static constexpr int OFF_CTRL = OFF_V + KV_STAGES * KV_BYTES;
  static constexpr int SMEM_BYTES = OFF_CTRL + 160;   // D=128: two CTAs (plus 1 KiB system reserve each) fit one SM
};
}  // namespace fp

static int make_tmap_tokens(CUtensorMap* out, const void* base, int64_t d, int64_t heads, int64_t tokens,
                            int64_t stride_h, int64_t stride_t, int box_tokens) {
  PFN_encodeTiled enc = get_encode_tiled();
  DLB_CHECK_ARG(enc != nullptr, DLB_ERR_DRIVER, "cuTensorMapEncodeTiled is not available from the driver");
  DLB_CHECK_ARG(((uintptr_t)base & 15) == 0, DLB_ERR_ALIGNMENT, "attention tensor base is not 16-byte aligned");
  DLB_CHECK_ARG((stride_h * 2) % 16 == 0 && (stride_t * 2) % 16 == 0, DLB_ERR_ALIGNMENT,
                "attention tensor strides must be multiples of 16 bytes");
  cuuint64_t dims[3] = {(cuuint64_t)d, (cuuint64_t)heads, (cuuint64_t)tokens};
  cuuint64_t strides[2] = {(cuuint64_t)stride_h * 2, (cuuint64_t)stride_t * 2};
  cuuint32_t box[3] = {64, 1, (cuuint32_t)box_tokens};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  DLB_CHECK_ARG(r == CUDA_SUCCESS, DLB_ERR_DRIVER, "cuTensorMapEncodeTiled(tokens) failed with CUresult %d", (int)r);
  return DLB_OK;
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(smem_dst)),
      "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// Packed pairs of fp32 in one 64-bit register (sm_100 f32x2 arithmetic)
__device__ __forceinline__ uint64_t pack_f2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack_f2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma_f2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add_f2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

struct PrefillParams {
  void* out;
  float* lse;                     // [hq, total] or null
  const int32_t* b_start_loc;
  const int32_t* b_seq_len;
  int64_t o_stride_t, o_stride_h;
  int64_t total_tokens;
  int batch, hq, hkv, group;
  int max_tiles;
  int causal;
  float scale_log2;               // sm_scale * log2(e)
  uint32_t idesc_qk, idesc_pv;
  uint32_t v_lbo, v_sbo;          // MN-major descriptor strides of the V tile
  int* status;
  // Paged K/V (prefill over a cache that already holds kv_seq_len - seq_len earlier tokens of each
  // sequence): tmap_k / tmap_v are then 4-D maps over [pages, slots, heads, d] and the keys of a
  // sequence are found through its row of the block table.
  int paged;
  int page_size, num_pages, max_pages;
  const void* block_table;        // [batch, max_pages] int32 or int64
  int64_t bt_stride;
  int table_is_int64;
  const int32_t* kv_seq_len;      // [batch]
  // Extras of the paged prefill branch (kernel instantiated with EXTRAS only when one is on):
  // Rotary embedding of Q inside the kernel (rotate-half convention, arithmetic in the 16-bit type): cos / sin
  // are [total_tokens, rot_dim] rows indexed like q's tokens; null = q is used as it is.  The Q tile is loaded
  // once per CTA, so its rotation is one pass of the softmax warps over the tile in shared memory; K is
  // expected to be rotated already (fill_kv_cache does it while it writes the cache).
  const void* rot_cos;
  const void* rot_sin;
  int rot_dim;
  int dv;                         // v / out head size (<= D, multiple of 8): output columns past it are not stored
  int window;                     // > 0: query at position pos sees keys pos - window .. pos (paged_attention.py:421-424,447)
  float softcap;                  // > 0: scores become softcap * tanh(score * sm_scale / softcap) (paged_attention.py:441-444)
  float sm_scale;
};

__device__ __forceinline__ int table_entry(const void* t, int64_t i, int is64) {
  return is64 ? (int)reinterpret_cast<const int64_t*>(t)[i] : reinterpret_cast<const int32_t*>(t)[i];
}

template <typename T, int D, bool EXTRAS>
__global__ void __launch_bounds__(fp::THREADS, 2)
flash_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                     const __grid_constant__ CUtensorMap tmap_v, const PrefillParams p) {
  using namespace fp;
  using L = Layout<D>;
  constexpr int BOXES = L::BOXES;
  constexpr int Q_BYTES = L::Q_BYTES, KV_BYTES = L::KV_BYTES;
  constexpr int OFF_Q = L::OFF_Q, OFF_K = L::OFF_K, OFF_V = L::OFF_V, OFF_CTRL = L::OFF_CTRL;
  // ---- which tile ----
  // CTA order: (sequence, kv head) groups one after the other; inside a group the heavy (late, causal)
  // tiles first, the q heads of the group adjacent.  The CTAs resident at any time then share the K/V
  // of one or two groups (4 MiB each at 8k tokens), which stay in L2 instead of being re-read from HBM.
  int x = blockIdx.x;
  const int hig = x % p.group;
  x /= p.group;
  const int tile = p.max_tiles - 1 - x % p.max_tiles;
  x /= p.max_tiles;
  const int kvh_ = x % p.hkv;
  const int seq = x / p.hkv;
  const int head = kvh_ * p.group + hig;
  const int seq_len = p.b_seq_len[seq];
  const int q0 = tile * BM;
  if (q0 >= seq_len) return;
  const int start = p.b_start_loc[seq];
  // query row r of the tile sits at position hist + q0 + r of its sequence (hist = tokens already cached)
  const int kv_len = p.paged ? p.kv_seq_len[seq] : seq_len;
  const int hist = kv_len - seq_len;
  const int kv_end = p.causal ? min(kv_len, q0 + BM + hist) : kv_len;
  // with a sliding window the tile starts at the block that holds the first key its first row may see;
  // `j` below counts blocks from there, jb0 + j is the block's index in the sequence
  const int jb0 = (EXTRAS && p.window > 0) ? max(0, q0 + hist - p.window) / BN : 0;
  const int nb = (kv_end + BN - 1) / BN - jb0;
  const int kvh = head / p.group;

  extern __shared__ __align__(1024) uint8_t smem[];
  if ((smem_u32(smem) & 1023u) != 0) {
    // the 128-byte swizzle needs 1 KiB aligned tiles; report instead of computing garbage
    if (threadIdx.x == 0 && p.status != nullptr && atomicCAS(p.status, 0, 2) == 0) p.status[1] = 20;
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OFF_CTRL);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;     // [2]
  uint64_t* v_full = bars + 5;     // [2]
  uint64_t* s_full = bars + 9;     // [2]
  // p_full is per S/P buffer: a fast softmax warp may finish block j+1 before a slow one finishes
  // block j, and its arrival must not count toward block j's phase
  uint64_t* p_full = bars + 11;    // [2]
  uint64_t* pv_done = bars + 13;   // [2] P.V of the block in S/P buffer s retired: V stage s reusable, O updated
  uint64_t* q_ready = bars + 15;   // Q tile rotated in place by the softmax warps (only with rot_cos)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    mbar_init(q_ready, 128);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&pv_done[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&p_full[i], 128);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  if (warp == WARP_MMA) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 128;

  if (warp == WARP_TMA) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
      mbar_arrive_expect_tx(q_full, Q_BYTES);
#pragma unroll
      for (int bx = 0; bx < BOXES; ++bx) tma_load_3d(smem + OFF_Q + bx * Q_BOX, &tmap_q, q_full, bx * 64, head, start + q0);
      // paged: the 64 keys of block j come from 64 / min(page, 64) pages of this sequence's table.  The
      // table entries of block j + 1 are fetched right after block j's K loads are issued, so that the
      // look-up's latency never sits between a freed stage and its next load.
      const int box_slots = min(p.page_size, BN);
      const int n_sub = p.paged ? BN / box_slots : 0;
      int pg[4] = {0, 0, 0, 0}, sl[4] = {0, 0, 0, 0};
      auto look_up = [&](int j) {
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (u >= n_sub) break;
          const int tok = (jb0 + j) * BN + u * box_slots;
          int page_slot = tok / p.page_size;
          if (page_slot >= p.max_pages) page_slot = p.max_pages - 1;   // past the table: any valid page, masked later
          int page = table_entry(p.block_table, (int64_t)seq * p.bt_stride + page_slot, p.table_is_int64);
          if (tok >= kv_len || page < 0 || page >= p.num_pages) page = 0;
          pg[u] = page;
          sl[u] = tok % p.page_size;
        }
      };
      if (nb > 0) look_up(0);
      for (int j = 0; j < nb; ++j) {
        const int s = j & 1;
        const uint32_t ph = (j >> 1) & 1;
        const int row = start + (jb0 + j) * BN;
        int pv[4], sv[4];   // block j's pages for the V loads below
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          pv[u] = pg[u];
          sv[u] = sl[u];
        }
        // K stage s is free once the Q K^T of block j - 2 has retired (s_full), V stage s once its P V has
        // (pv_done): no separate "empty" commits, every commit costs the single issuing thread ~100 clocks
        if (!mbar_wait(&s_full[s], ph ^ 1, abort_flag, p.status, 21, j)) break;
        uint8_t* kd = smem + OFF_K + s * KV_BYTES;
        mbar_arrive_expect_tx(&k_full[s], KV_BYTES);
        if (p.paged) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (u >= n_sub) break;
#pragma unroll
            for (int bx = 0; bx < BOXES; ++bx)
              tma_load_4d(kd + bx * KV_BOX + u * box_slots * 128, &tmap_k, &k_full[s], bx * 64, kvh, sl[u], pg[u]);
          }
        } else {
#pragma unroll
          for (int bx = 0; bx < BOXES; ++bx) tma_load_3d(kd + bx * KV_BOX, &tmap_k, &k_full[s], bx * 64, kvh, row);
        }
        if (j + 1 < nb) look_up(j + 1);
        if (!mbar_wait(&pv_done[s], ph ^ 1, abort_flag, p.status, 22, j)) break;
        uint8_t* vd = smem + OFF_V + s * KV_BYTES;
        mbar_arrive_expect_tx(&v_full[s], KV_BYTES);
        if (p.paged) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            if (u >= n_sub) break;
#pragma unroll
            for (int bx = 0; bx < BOXES; ++bx)
              tma_load_4d(vd + bx * KV_BOX + u * box_slots * 128, &tmap_v, &v_full[s], bx * 64, kvh, sv[u], pv[u]);
          }
        } else {
#pragma unroll
          for (int bx = 0; bx < BOXES; ++bx) tma_load_3d(vd + bx * KV_BOX, &tmap_v, &v_full[s], bx * 64, kvh, row);
        }
      }
    }
  } else if (warp == WARP_MMA) {
    // ------------------------------ MMA issuer ------------------------------
    if (lane == 0) {
      bool ok = mbar_wait(p.rot_cos != nullptr ? q_ready : q_full, 0, abort_flag, p.status, 23, 0);
      if (p.rot_cos != nullptr) tc_fence_after_sync();
      // descriptors as (low, high) words: only the address field (bytes >> 4) in the low word moves
      const uint64_t q_d0 = make_smem_desc(smem_u32(smem + OFF_Q), 16, 1024, 2);
      const uint64_t k_d0 = make_smem_desc(smem_u32(smem + OFF_K), 16, 1024, 2);
      const uint64_t v_d0 = make_smem_desc(smem_u32(smem + OFF_V), p.v_lbo, p.v_sbo, 2);
      const uint32_t q_lo0 = (uint32_t)q_d0, k_lo0 = (uint32_t)k_d0, kq_hi = (uint32_t)(q_d0 >> 32);
      const uint32_t v_lo0 = (uint32_t)v_d0, v_hi = (uint32_t)(v_d0 >> 32);
      for (int j = 0; ok && j <= nb; ++j) {
        if (j < nb) {
          // S_j = Q K_j^T
          const int s = j & 1;
          const uint32_t ph = (j >> 1) & 1;
          if (!mbar_wait(&k_full[s], ph, abort_flag, p.status, 24, j)) { ok = false; break; }
          // S buffer s also carried P_{j-2}: P_{j-2} V_{j-2} was issued before this MMA and the tensor
          // pipe runs one thread's MMAs in order, so no barrier is needed before overwriting it
          tc_fence_after_sync();
          const uint32_t k_lo = k_lo0 + (uint32_t)s * (KV_BYTES >> 4);
#pragma unroll
          for (int ks = 0; ks < D / 16; ++ks) {
            const uint32_t off = (uint32_t)(((ks >> 2) * Q_BOX + (ks & 3) * 32) >> 4);
            const uint32_t koff = (uint32_t)(((ks >> 2) * KV_BOX + (ks & 3) * 32) >> 4);
            if (ks == 0) umma_ss_lohi<0>(tmem_base + s * BN, q_lo0 + off, kq_hi, k_lo + koff, kq_hi, p.idesc_qk);
            else umma_ss_lohi<1>(tmem_base + s * BN, q_lo0 + off, kq_hi, k_lo + koff, kq_hi, p.idesc_qk);
          }
          umma_commit(&s_full[s]);
        }
        if (j > 0) {
          // O += P_{j-1} V_{j-1}
          const int jj = j - 1;
          const int s = jj & 1;
          const uint32_t ph = (jj >> 1) & 1;
          {
            // poll both barriers at once (their latencies overlap); wait in turn only if one is not ready
            const bool r1 = mbar_try_wait(&p_full[s], ph), r2 = mbar_try_wait(&v_full[s], ph);
            if (!(r1 && r2)) {
              if (!mbar_wait(&p_full[s], ph, abort_flag, p.status, 26, jj)) { ok = false; break; }
              if (!mbar_wait(&v_full[s], ph, abort_flag, p.status, 27, jj)) { ok = false; break; }
            }
          }
          tc_fence_after_sync();
          const uint32_t v_lo = v_lo0 + (uint32_t)s * (KV_BYTES >> 4);
          // A = P_{jj} from TMEM (16-bit pairs in the first 32 columns of S buffer s), 8 columns per K16 step
          if (jj == 0) umma_ts_lohi<0>(tmem_o, tmem_base + s * BN, v_lo, v_hi, p.idesc_pv);
          else umma_ts_lohi<1>(tmem_o, tmem_base + s * BN, v_lo, v_hi, p.idesc_pv);
#pragma unroll
          for (int ks = 1; ks < BN / 16; ++ks)
            umma_ts_lohi<1>(tmem_o, tmem_base + s * BN + ks * 8, v_lo + ks * (16 * 128 >> 4), v_hi, p.idesc_pv);
          umma_commit(&pv_done[s]);
        }
      }
    }
  } else if (warp < 4) {
    // ------------------------------ softmax / correction / epilogue ------------------------------
    const int quad = warp;
    const int row = quad * 32 + lane;              // query row inside the tile == TMEM lane
    const int q_pos = q0 + row;                    // position inside the sequence
    const uint32_t lane_field = (uint32_t)(quad * 32) << 16;
    float m_ref = -CUDART_INF_F;                   // reference max used for exponentiation (scaled, log2 domain)
    float l_sum = 0.f;
    bool ok = true;
    if (p.rot_cos != nullptr) {
      // rotate this thread's query row in place in the swizzled Q tile (16-byte chunk c of row r sits at chunk
      // position c ^ (r & 7) of its 128-byte line), then hand the tile to the MMA thread.  The row's cos / sin
      // values are fetched BEFORE the wait for the Q tile, so the two latencies overlap.
      const bool row_live = q_pos < seq_len;
      const int half = p.rot_dim >> 1, hv = half >> 3;          // hv <= 8 (head size <= 128)
      const T* cs = reinterpret_cast<const T*>(p.rot_cos) + (int64_t)(start + (row_live ? q_pos : 0)) * p.rot_dim;
      const T* sn = reinterpret_cast<const T*>(p.rot_sin) + (int64_t)(start + (row_live ? q_pos : 0)) * p.rot_dim;
      uint4 cl[8], ch[8], sl[8], sh[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (i < hv && row_live) {
          cl[i] = __ldg(reinterpret_cast<const uint4*>(cs) + i);
          ch[i] = __ldg(reinterpret_cast<const uint4*>(cs + half) + i);
          sl[i] = __ldg(reinterpret_cast<const uint4*>(sn) + i);
          sh[i] = __ldg(reinterpret_cast<const uint4*>(sn + half) + i);
        }
      }
      ok = mbar_wait(q_full, 0, abort_flag, p.status, 32, 0);
      ok = __all_sync(0xffffffffu, ok);
      if (ok && row_live) {
        auto chunk_at = [&](int col) -> uint4* {
          return reinterpret_cast<uint4*>(smem + OFF_Q + (col >> 6) * Q_BOX + row * 128 +
                                          ((((col & 63) >> 3) ^ (row & 7)) << 4));
        };
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if (i < hv) {
            uint4* plo = chunk_at(i * 8);
            uint4* phi = chunk_at(half + i * 8);
            uint4 olo, ohi;
            rot_vec8<T>(*plo, *phi, cl[i], ch[i], sl[i], sh[i], olo, ohi);
            *plo = olo;
            *phi = ohi;
          }
        }
      }
      fence_proxy_async_smem();     // generic-proxy stores before the tensor core's reads of the tile
      mbar_arrive(q_ready);
    }
    for (int j = 0; ok && j < nb; ++j) {
      const int s = j & 1;
      const uint32_t ph = (j >> 1) & 1;
      ok = mbar_wait(&s_full[s], ph, abort_flag, p.status, 28, j);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      tc_fence_after_sync();
      uint32_t sr[2][32];
      tmem_ld_32x32b_x32(tmem_base + lane_field + s * BN, sr[0]);
      tmem_ld_32x32b_x32(tmem_base + lane_field + s * BN + 32, sr[1]);
      tmem_wait_ld();

      // soft-cap: the scores go to the log2 domain here (cap * tanh(s * sm_scale / cap) * log2 e) and the scale
      // applied further down becomes 1
      float eff_scale = p.scale_log2;
      if (EXTRAS && p.softcap > 0.f) {
        const float inv = p.sm_scale / p.softcap, capl2 = p.softcap * 1.4426950408889634f;
#pragma unroll
        for (int h = 0; h < 2; ++h)
#pragma unroll
          for (int c = 0; c < 32; ++c)
            sr[h][c] = __float_as_uint(capl2 * tanhf(__uint_as_float(sr[h][c]) * inv));
        eff_scale = 1.f;
      }
      // mask (diagonal / tail / window-edge blocks only)
      const int key0 = (jb0 + j) * BN;
      const int win_lo = (EXTRAS && p.window > 0) ? q_pos + hist - p.window : -(1 << 30);   // first visible key
      const bool need_mask = (key0 + BN > kv_end) || (p.causal && key0 + BN - 1 > q0 + hist) ||
                             (EXTRAS && p.window > 0 && key0 < q0 + BM + hist - p.window);
      if (need_mask) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
#pragma unroll
          for (int c = 0; c < 32; ++c) {
            const int key = key0 + h * 32 + c;
            const bool visible = key < kv_end && (!p.causal || key <= q_pos + hist) && key >= win_lo;
            if (!visible) sr[h][c] = 0xff800000u;   // -inf
          }
        }
      }
      // row max of the raw scores (3-input max), scaled once: scale > 0 keeps the order
      float mx4[4] = {-CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F, -CUDART_INF_F};   // 4 independent chains
#pragma unroll
      for (int h = 0; h < 2; ++h) {
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            mx4[u] = max3(mx4[u], __uint_as_float(sr[h][c + 2 * u]), __uint_as_float(sr[h][c + 2 * u + 1]));
        }
      }
      float mx = fmaxf(max3(mx4[0], mx4[1], mx4[2]), mx4[3]);
      mx *= eff_scale;
      // lazy rescale decision
      float alpha = 1.f;
      bool rescale = false;
      if (m_ref == -CUDART_INF_F) {
        m_ref = mx;                                 // first visible block: nothing accumulated yet
      } else if (mx - m_ref > RESCALE_THRESHOLD) {
        alpha = fast_exp2(m_ref - mx);
        m_ref = mx;
        rescale = true;
      }
      // O may be rescaled only once P_{j-1} V_{j-1} has retired.  (P_{j-2} V_{j-2} retired before S_j was
      // signalled, so the barrier is never more than one phase behind and the parity wait is exact.)
      if (j > 0 && __any_sync(0xffffffffu, rescale)) {
        ok = mbar_wait(&pv_done[(j - 1) & 1], ((j - 1) >> 1) & 1, abort_flag, p.status, 29, j);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        tc_fence_after_sync();
        {
#pragma unroll 1
          for (int c = 0; c < D / 32; ++c) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(tmem_o + lane_field + c * 32, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32b_x32(tmem_o + lane_field + c * 32, o);
          }
          tmem_wait_st();
        }
      }
      // p = 2^(s * scale - m): one packed FMA per two scores, exponentials on the SFU, packed adds for
      // the row sum, one conversion per pair; each half row (32 scores -> 16 packed registers) goes
      // back to TMEM over the first columns of the S buffer it came from, where the P.V MMA reads it
      // as its A operand
      const float neg_m = (m_ref == -CUDART_INF_F) ? 0.f : -m_ref;
      const uint64_t scale2 = pack_f2(eff_scale, eff_scale);
      const uint64_t negm2 = pack_f2(neg_m, neg_m);
      uint64_t sum2a = pack_f2(0.f, 0.f), sum2b = sum2a;
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        uint32_t pk[16];
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          const uint64_t a01 =
              fma_f2(pack_f2(__uint_as_float(sr[h][c]), __uint_as_float(sr[h][c + 1])), scale2, negm2);
          const uint64_t a23 =
              fma_f2(pack_f2(__uint_as_float(sr[h][c + 2]), __uint_as_float(sr[h][c + 3])), scale2, negm2);
          float x0, x1, x2, x3;
          unpack_f2(a01, x0, x1);
          unpack_f2(a23, x2, x3);
          const float e0 = fast_exp2(x0), e1 = fast_exp2(x1), e2 = fast_exp2(x2), e3 = fast_exp2(x3);
          sum2a = add_f2(sum2a, pack_f2(e0, e1));
          sum2b = add_f2(sum2b, pack_f2(e2, e3));
          typename Elem<T>::T2 v01 = Elem<T>::from_f2(e0, e1);
          typename Elem<T>::T2 v23 = Elem<T>::from_f2(e2, e3);
          pk[c / 2] = *reinterpret_cast<uint32_t*>(&v01);
          pk[c / 2 + 1] = *reinterpret_cast<uint32_t*>(&v23);
        }
        tmem_st_32x32b_x16(tmem_base + lane_field + s * BN + h * 16, pk);
      }
      {
        float a, b;
        unpack_f2(add_f2(sum2a, sum2b), a, b);
        l_sum = l_sum * alpha + (a + b);
      }
      if (key0 + BN > kv_len) {
        // rows of this V tile past the last key: zero them (generic-proxy stores), then make the stores
        // visible to the tensor core's shared-memory reads before this block's P.V can be issued
        ok = mbar_wait(&v_full[s], ph, abort_flag, p.status, 31, j);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        const int first_dead = max(kv_len - key0, 0);
        uint8_t* vt = smem + OFF_V + s * KV_BYTES;
        for (int i = threadIdx.x; i < (BN - first_dead) * BOXES * 8; i += 128) {
          const int chunk = i & 7, bx = (i >> 3) % BOXES, r = first_dead + (i >> 3) / BOXES;
          *reinterpret_cast<uint4*>(vt + bx * KV_BOX + r * 128 + chunk * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        fence_proxy_async_smem();
      }
      tmem_wait_st();
      tc_fence_before_sync();
      mbar_arrive(&p_full[s]);
    }
    if (ok) {
      // the last P.V (the one before it in the same buffer, block nb - 3, retired before S of block nb - 1
      // was signalled, so the parity is exact)
      ok = mbar_wait(&pv_done[(nb - 1) & 1], ((nb - 1) >> 1) & 1, abort_flag, p.status, 30, nb);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      tc_fence_after_sync();
      const float inv_l = 1.f / l_sum;
      const bool row_ok = q_pos < seq_len;
      T* orow = reinterpret_cast<T*>(p.out) + (int64_t)(start + q_pos) * p.o_stride_t + (int64_t)head * p.o_stride_h;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld_32x32b_x32(tmem_o + lane_field + c * 32, o);
        tmem_wait_ld();
        if (row_ok) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              typename Elem<T>::T2 v2 = Elem<T>::from_f2(__uint_as_float(o[v * 8 + 2 * i]) * inv_l,
                                                         __uint_as_float(o[v * 8 + 2 * i + 1]) * inv_l);
              w[i] = *reinterpret_cast<uint32_t*>(&v2);
            }
            if (c * 32 + v * 8 < p.dv)
              *reinterpret_cast<uint4*>(orow + c * 32 + v * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      if (row_ok && p.lse != nullptr) {
        p.lse[(int64_t)head * p.total_tokens + start + q_pos] = m_ref * 0.6931471805599453f + __logf(l_sum);
      }
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == WARP_MMA) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <typename T, int D, bool EXTRAS>
static int launch_prefill_x(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                            const PrefillParams& p, unsigned grid, cudaStream_t stream) {
  auto kern = flash_prefill_kernel<T, D, EXTRAS>;
  constexpr int SMEM = fp::Layout<D>::SMEM_BYTES;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) {
    set_last_error("flash_prefill: smem attribute: %s", cudaGetErrorString(e));
    return (int)e;
  }
  kern<<<grid, fp::THREADS, SMEM, stream>>>(tq, tk, tv, p);
  return DLB_OK;
}
template <typename T, int D>
static int launch_prefill(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const PrefillParams& p,
                          unsigned grid, cudaStream_t stream) {
  return (p.window > 0 || p.softcap > 0.f) ? launch_prefill_x<T, D, true>(tq, tk, tv, p, grid, stream)
                                           : launch_prefill_x<T, D, false>(tq, tk, tv, p, grid, stream);
}

}  // namespace dlb

extern "C" int dlb_flash_prefill_varlen(const void* q, const void* k, const void* v, void* out, float* lse,
                                        const int32_t* b_start_loc, const int32_t* b_seq_len, int64_t batch,
                                        int64_t total_tokens, int64_t max_seq_len, int64_t hq, int64_t hkv,
                                        int64_t head_dim, int64_t head_dim_v, int64_t q_stride_t, int64_t q_stride_h,
                                        int64_t k_stride_t, int64_t k_stride_h, int64_t v_stride_t,
                                        int64_t v_stride_h, int64_t o_stride_t, int64_t o_stride_h, float sm_scale,
                                        int causal, const void* q_cos, const void* q_sin, int dtype, int32_t* status,
                                        void* stream) {
  DLB_NVTX("dlb_flash_prefill_varlen");
  using namespace dlb;
  using namespace dlb::fp;
  DLB_CHECK_ARG(dtype == DLB_DTYPE_BF16 || dtype == DLB_DTYPE_F16, DLB_ERR_UNSUPPORTED,
                "flash_prefill: dtype %d (need fp16 or bf16)", dtype);
  DLB_CHECK_ARG(head_dim >= 8 && head_dim <= 128 && head_dim % 8 == 0 && head_dim_v >= 8 && head_dim_v <= 128 &&
                    head_dim_v % 8 == 0,
                DLB_ERR_UNSUPPORTED, "flash_prefill: head_dim %lld / %lld not supported (multiples of 8 up to 128)",
                (long long)head_dim, (long long)head_dim_v);
  const int D = (head_dim <= 64 && head_dim_v <= 64) ? 64 : 128;   // tile width; the tensor maps keep the true sizes
  DLB_CHECK_ARG(batch >= 0 && hq >= 1 && hkv >= 1 && hq % hkv == 0, DLB_ERR_BAD_ARG, "flash_prefill: bad head counts");
  DLB_CHECK_ARG(total_tokens >= 0 && max_seq_len >= 0, DLB_ERR_BAD_ARG, "flash_prefill: negative size");
  if (batch == 0 || total_tokens == 0 || max_seq_len == 0) return DLB_OK;
  DLB_CHECK_ARG(q && k && v && out && b_start_loc && b_seq_len, DLB_ERR_BAD_ARG, "flash_prefill: null pointer");
  DLB_CHECK_ARG(((uintptr_t)out & 15) == 0 && o_stride_t % 8 == 0 && o_stride_h % 8 == 0, DLB_ERR_ALIGNMENT,
                "flash_prefill: output must be 16-byte aligned with strides that are multiples of 8");
  const int64_t max_tiles = (max_seq_len + BM - 1) / BM;
  const int64_t grid = max_tiles * batch * hq;
  DLB_CHECK_ARG(grid <= 0x7fffffffLL && total_tokens < (1LL << 31), DLB_ERR_TOO_LARGE, "flash_prefill: grid too large");

  const int kv_box = BN;
  CUtensorMap tq, tk, tv;
  int rc = make_tmap_tokens(&tq, q, head_dim, hq, total_tokens, q_stride_h, q_stride_t, BM);
  if (rc != DLB_OK) return rc;
  rc = make_tmap_tokens(&tk, k, head_dim, hkv, total_tokens, k_stride_h, k_stride_t, kv_box);
  if (rc != DLB_OK) return rc;
  rc = make_tmap_tokens(&tv, v, head_dim_v, hkv, total_tokens, v_stride_h, v_stride_t, kv_box);
  if (rc != DLB_OK) return rc;

  const uint32_t fmt = dtype == DLB_DTYPE_BF16 ? 1u : 0u;
  PrefillParams p;
  p.out = out;
  p.lse = lse;
  p.b_start_loc = b_start_loc;
  p.b_seq_len = b_seq_len;
  p.o_stride_t = o_stride_t;
  p.o_stride_h = o_stride_h;
  p.total_tokens = total_tokens;
  p.batch = (int)batch;
  p.hq = (int)hq;
  p.hkv = (int)hkv;
  p.group = (int)(hq / hkv);
  p.max_tiles = (int)max_tiles;
  p.causal = causal;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.idesc_qk = make_idesc_f16(BM, kv_box, fmt, 0u, 0u);
  p.idesc_pv = make_idesc_f16(BM, D, fmt, 0u, 1u);
  // V tile in shared memory: two 64-wide (128 B) column boxes of BN key rows each.
  // MN-major canonical layout: 64 d contiguous, next 64-d atom at LBO; 8 key rows at
  // 128 B pitch, next group of 8 keys at SBO.
  p.v_lbo = KV_BOX;
  p.v_sbo = 1024;
  p.status = status;
  p.paged = 0;
  p.page_size = BN;
  p.num_pages = p.max_pages = 0;
  p.block_table = nullptr;
  p.bt_stride = 0;
  p.table_is_int64 = 0;
  p.kv_seq_len = nullptr;
  DLB_CHECK_ARG((q_cos == nullptr) == (q_sin == nullptr), DLB_ERR_BAD_ARG, "flash_prefill: cos and sin go together");
  DLB_CHECK_ARG(q_cos == nullptr || (head_dim % 16 == 0 && (((uintptr_t)q_cos | (uintptr_t)q_sin) & 15) == 0),
                DLB_ERR_ALIGNMENT, "flash_prefill: rotary needs a head size that is a multiple of 16 and 16-byte aligned cos / sin");
  p.rot_cos = q_cos;
  p.rot_sin = q_sin;
  p.rot_dim = (int)head_dim;
  p.dv = (int)head_dim_v;
  p.window = 0;
  p.softcap = 0.f;
  p.sm_scale = sm_scale;

  cudaStream_t s = (cudaStream_t)stream;
  int rc2;
  if (dtype == DLB_DTYPE_BF16) {
    rc2 = D == 128 ? launch_prefill<__nv_bfloat16, 128>(tq, tk, tv, p, (unsigned)grid, s)
                   : launch_prefill<__nv_bfloat16, 64>(tq, tk, tv, p, (unsigned)grid, s);
  } else {
    rc2 = D == 128 ? launch_prefill<__half, 128>(tq, tk, tv, p, (unsigned)grid, s)
                   : launch_prefill<__half, 64>(tq, tk, tv, p, (unsigned)grid, s);
  }
  if (rc2 != DLB_OK) return rc2;
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}

extern "C" int dlb_flash_prefill_paged(const void* q, const void* k_cache, const void* v_cache, void* out, float* lse,
                                       const void* block_table, const int32_t* q_start_loc,
                                       const int32_t* q_seq_len, const int32_t* kv_seq_len, int64_t batch,
                                       int64_t total_q_tokens, int64_t max_q_len, int64_t hq, int64_t hkv,
                                       int64_t head_dim, int64_t head_dim_v, int64_t page_size, int64_t num_pages,
                                       int64_t max_pages,
                                       int64_t q_stride_t, int64_t q_stride_h, int64_t k_stride_page,
                                       int64_t k_stride_slot, int64_t k_stride_head, int64_t v_stride_page,
                                       int64_t v_stride_slot, int64_t v_stride_head, int64_t o_stride_t,
                                       int64_t o_stride_h, int64_t bt_stride, int table_is_int64, int64_t window,
                                       float sm_scale, float softcap, int causal, const void* q_cos,
                                       const void* q_sin, int dtype, int32_t* status, void* stream) {
  DLB_NVTX("dlb_flash_prefill_paged");
  using namespace dlb;
  using namespace dlb::fp;
  DLB_CHECK_ARG(dtype == DLB_DTYPE_BF16 || dtype == DLB_DTYPE_F16, DLB_ERR_UNSUPPORTED,
                "flash_prefill_paged: dtype %d (need fp16 or bf16)", dtype);
  DLB_CHECK_ARG(head_dim >= 8 && head_dim <= 128 && head_dim % 8 == 0 && head_dim_v >= 8 && head_dim_v <= 128 &&
                    head_dim_v % 8 == 0,
                DLB_ERR_UNSUPPORTED,
                "flash_prefill_paged: head_dim %lld / %lld not supported (multiples of 8 up to 128)",
                (long long)head_dim, (long long)head_dim_v);
  const int D = (head_dim <= 64 && head_dim_v <= 64) ? 64 : 128;   // tile width; the tensor maps keep the true sizes
  DLB_CHECK_ARG(batch >= 0 && hq >= 1 && hkv >= 1 && hq % hkv == 0, DLB_ERR_BAD_ARG,
                "flash_prefill_paged: bad head counts");
  DLB_CHECK_ARG(total_q_tokens >= 0 && max_q_len >= 0, DLB_ERR_BAD_ARG, "flash_prefill_paged: negative size");
  DLB_CHECK_ARG(page_size >= 16 && (page_size & (page_size - 1)) == 0, DLB_ERR_UNSUPPORTED,
                "flash_prefill_paged: page size %lld must be a power of two >= 16", (long long)page_size);
  DLB_CHECK_ARG(num_pages >= 1 && max_pages >= 1, DLB_ERR_BAD_ARG, "flash_prefill_paged: empty cache or table");
  if (batch == 0 || total_q_tokens == 0 || max_q_len == 0) return DLB_OK;
  DLB_CHECK_ARG(q && k_cache && v_cache && out && block_table && q_start_loc && q_seq_len && kv_seq_len,
                DLB_ERR_BAD_ARG, "flash_prefill_paged: null pointer");
  DLB_CHECK_ARG(((uintptr_t)out & 15) == 0 && o_stride_t % 8 == 0 && o_stride_h % 8 == 0, DLB_ERR_ALIGNMENT,
                "flash_prefill_paged: output must be 16-byte aligned with strides that are multiples of 8");
  const int64_t max_tiles = (max_q_len + BM - 1) / BM;
  const int64_t grid = max_tiles * batch * hq;
  DLB_CHECK_ARG(grid <= 0x7fffffffLL && total_q_tokens < (1LL << 31), DLB_ERR_TOO_LARGE,
                "flash_prefill_paged: grid too large");

  CUtensorMap tq, tk, tv;
  int rc = make_tmap_tokens(&tq, q, head_dim, hq, total_q_tokens, q_stride_h, q_stride_t, BM);
  if (rc != DLB_OK) return rc;
  const int box_slots = (int)(page_size < BN ? page_size : BN);
  rc = make_tmap_cache(&tk, k_cache, head_dim, hkv, page_size, num_pages, k_stride_page, k_stride_slot,
                       k_stride_head, box_slots);
  if (rc != DLB_OK) return rc;
  rc = make_tmap_cache(&tv, v_cache, head_dim_v, hkv, page_size, num_pages, v_stride_page, v_stride_slot,
                       v_stride_head, box_slots);
  if (rc != DLB_OK) return rc;

  const uint32_t fmt = dtype == DLB_DTYPE_BF16 ? 1u : 0u;
  PrefillParams p;
  p.out = out;
  p.lse = lse;
  p.b_start_loc = q_start_loc;
  p.b_seq_len = q_seq_len;
  p.o_stride_t = o_stride_t;
  p.o_stride_h = o_stride_h;
  p.total_tokens = total_q_tokens;
  p.batch = (int)batch;
  p.hq = (int)hq;
  p.hkv = (int)hkv;
  p.group = (int)(hq / hkv);
  p.max_tiles = (int)max_tiles;
  p.causal = causal;
  p.scale_log2 = sm_scale * 1.4426950408889634f;
  p.idesc_qk = make_idesc_f16(BM, BN, fmt, 0u, 0u);
  p.idesc_pv = make_idesc_f16(BM, D, fmt, 0u, 1u);
  p.v_lbo = KV_BOX;
  p.v_sbo = 1024;
  p.status = status;
  p.paged = 1;
  p.page_size = (int)page_size;
  p.num_pages = (int)num_pages;
  p.max_pages = (int)max_pages;
  p.block_table = block_table;
  p.bt_stride = bt_stride;
  p.table_is_int64 = table_is_int64;
  p.kv_seq_len = kv_seq_len;
  DLB_CHECK_ARG((q_cos == nullptr) == (q_sin == nullptr), DLB_ERR_BAD_ARG,
                "flash_prefill_paged: cos and sin go together");
  DLB_CHECK_ARG(q_cos == nullptr || (head_dim % 16 == 0 && (((uintptr_t)q_cos | (uintptr_t)q_sin) & 15) == 0),
                DLB_ERR_ALIGNMENT,
                "flash_prefill_paged: rotary needs a head size that is a multiple of 16 and 16-byte aligned cos / sin");
  p.rot_cos = q_cos;
  p.rot_sin = q_sin;
  p.rot_dim = (int)head_dim;
  p.dv = (int)head_dim_v;
  p.window = window > 0 ? (int)std::min<int64_t>(window, 1 << 29) : 0;
  p.softcap = softcap;
  p.sm_scale = sm_scale;

  cudaStream_t s = (cudaStream_t)stream;
  int rc2;
  if (dtype == DLB_DTYPE_BF16) {
    rc2 = D == 128 ? launch_prefill<__nv_bfloat16, 128>(tq, tk, tv, p, (unsigned)grid, s)
                   : launch_prefill<__nv_bfloat16, 64>(tq, tk, tv, p, (unsigned)grid, s);
  } else {
    rc2 = D == 128 ? launch_prefill<__half, 128>(tq, tk, tv, p, (unsigned)grid, s)
                   : launch_prefill<__half, 64>(tq, tk, tv, p, (unsigned)grid, s);
  }
  if (rc2 != DLB_OK) return rc2;
  DLB_CUDA_LAUNCH_CHECK();
  return DLB_OK;
}
