// Paged flash-decode: one query token per sequence against a paged KV cache,
// split over the KV length, with a log-sum-exp merge.
//
// Same math as the reference's split-K decode path
// (python/dlBLAS/dlblas/kernels/paged_attention.py:40-285): scores
// q.k * sm_scale (optional tanh soft-cap, optional sliding window), online
// softmax in fp32, P cast to the cache dtype before P.V, per-split partial
// (acc, m, l) merged by rescaling with exp(m_s - m_max).  Differences are
// structural only: the number of splits adapts to each sequence's length
// (fixed `chunk` tokens per split instead of a fixed 4 splits), so a batch that
// mixes 1k and 32k contexts keeps every SM busy.
//
// HBM-bound (about 4 FLOP per byte of KV), so the kernel is built around the
// memory system: a producer lane walks the block table and issues TMA tile
// loads (4-D tensor map over [page, slot, kv-head, d], 128-byte swizzle) into a
// multi-stage shared-memory ring guarded by mbarriers; four consumer warps each
// own 16 of the 64 keys of a tile and run mma.sync m16n8k16 with the
// sequence's q-heads of one kv-head as the (zero-padded) M=16 rows, fed by
// swizzle-aware ldmatrix.  Each KV byte is read from HBM exactly once.
//
// The kernel is built for tile widths D = 64 and 128.  Any q/k head size and any v head size that are
// multiples of 8 up to 128 run on the next width (the reference splits the head into a power of two plus a
// remainder and lets V have its own size, paged_attention.py:526-539): the tensor maps carry the TRUE
// sizes, so the copy engine fills the missing columns of every tile with zeros in shared memory (no copy of
// the cache), zero columns add nothing to a score, and output columns past the v head size are not stored.
#include <math_constants.h>

#include <mutex>

#include "common.cuh"

namespace dlb {

namespace pd {
constexpr int TILE_KEYS = 64;
constexpr int CONSUMER_WARPS = 4;
constexpr int THREADS = 32 * (CONSUMER_WARPS + 1);
constexpr int GATHER_WARPS = 4;                 // producer warps when rows are gathered with cp.async
constexpr int GATHER_ROWS = 64 / GATHER_WARPS;  // rows of a 64-key tile per producer warp
constexpr int STAGES = 3;
}  // namespace pd

__device__ __forceinline__ void ldmatrix_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2,
                                                  uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
               : "r"(addr));
}
template <typename T>
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma_16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                         uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma_16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
      "{%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <typename T> __device__ __forceinline__ uint32_t pack_pair(float a, float b);
template <> __device__ __forceinline__ uint32_t pack_pair<__nv_bfloat16>(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack_pair<__half>(float a, float b) {
  __half2 v = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

struct DecodeParams {
  const void* q;             // [B, Hq, D]
  void* out;                 // [B, Hq, D]
  float* partial;            // [B, Hq, max_splits, D + 2] fp32 (acc, m, l); unused when max_splits == 1
  const void* block_table;   // [B, max_pages] int32 or int64
  const void* kv_seqlens;    // [B] int32 or int64
  int64_t q_stride_b, q_stride_h;
  int64_t o_stride_b, o_stride_h;
  int64_t bt_stride;
  int batch, hq, hkv, group;
  int dk, dv;                // true head sizes of q/k and of v/out (<= D, multiples of 8); columns beyond them are zero
  int page_size, max_pages, num_pages;
  int chunk;                 // tokens per split (multiple of 64 and of the page size when page_size > 64)
  int max_splits;
  int window;                // <= 0: none
  int table_is_int64, lens_is_int64;
  float sm_scale, softcap;   // softcap <= 0: none
  int* status;
  // gather path (pages smaller than 8 tokens): plain pointers and element strides of the caches
  int gather;
  const void* k_cache;
  const void* v_cache;
  int64_t k_stride_head, v_stride_head;                   // elements
  uint32_t k_page_bytes, k_slot_bytes, v_page_bytes, v_slot_bytes;
  int page_shift;                                         // log2(page_size) in the gather path (1, 2 or 4 tokens)
};

// 16-byte asynchronous copy global -> shared (bypassing L1), or 16 bytes of zeros when src_bytes == 0 (a
// chunk past the head size: the zero fill stays inside the cp.async group, so the stage's barrier covers
// it like any other chunk), to `smem_dst + DST_OFFSET`: the offset is an immediate of the instruction, so
// one address register serves the K and the V half of a stage.  cp_async_arrive: "arrive on this mbarrier
// once all of this thread's earlier cp.async copies have landed" (one of the barrier's expected count).
template <int DST_OFFSET>
__device__ __forceinline__ void cp_async_16_sized(uint32_t smem_dst, const void* gmem_src, uint32_t src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0 + %3], [%1], 16, %2;" ::"r"(smem_dst), "l"(gmem_src), "r"(src_bytes),
               "n"(DST_OFFSET)
               : "memory");
}
__device__ __forceinline__ void cp_async_arrive(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ int load_index(const void* p, int64_t i, int is64) {
  return is64 ? (int)reinterpret_cast<const int64_t*>(p)[i] : reinterpret_cast<const int32_t*>(p)[i];
}

// Token range [lo, hi) of split `s`; returns false if the split is empty.
__device__ __forceinline__ bool split_range(int ctx, int window, int chunk, int s, int& lo, int& hi, int& kv_lo) {
  // the query sits at position ctx - 1 and sees keys ctx - 1 - window .. ctx - 1, as in the reference
  // (paged_attention.py:163-165,192-194 with history_len = ctx - 1)
  kv_lo = (window > 0 && ctx - 1 > window) ? ctx - 1 - window : 0;
  const int base = (kv_lo / pd::TILE_KEYS) * pd::TILE_KEYS;
  lo = base + s * chunk;
  hi = min(ctx, lo + chunk);
  return lo < hi;
}

template <typename T, int D>
__global__ void __launch_bounds__(pd::THREADS + 32 * (pd::GATHER_WARPS - 1), 2)
paged_decode_split_kernel(const __grid_constant__ CUtensorMap tmap_k, const __grid_constant__ CUtensorMap tmap_v,
                          const DecodeParams p) {
  using namespace pd;
  constexpr int HALF_BYTES = TILE_KEYS * 128;         // one 64-key x 64-d swizzled box
  constexpr int BOXES = D / 64;
  constexpr int KV_BYTES = BOXES * HALF_BYTES;        // K (or V) tile
  constexpr int STAGE_BYTES = 2 * KV_BYTES;
  constexpr int KSTEPS = D / 16;
  constexpr int NT = D / 8;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw_addr = smem_u32(smem_raw);
  uint8_t* smem = smem_raw + (((raw_addr + 1023u) & ~1023u) - raw_addr);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + STAGES * STAGE_BYTES);
  uint64_t* empty_bar = full_bar + STAGES;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(empty_bar + STAGES);

  const int split = blockIdx.x;
  const int kvh = blockIdx.y % p.hkv;
  const int hblk = blockIdx.y / p.hkv;          // block of 16 q-heads inside the group
  const int b = blockIdx.z;
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int ctx = load_index(p.kv_seqlens, b, p.lens_is_int64);
  int lo, hi, kv_lo;
  if (!split_range(ctx, p.window, p.chunk, split, lo, hi, kv_lo)) {
    // empty split: nothing to do, except that without a merge pass an empty context still owes zeros
    if (p.max_splits == 1) {
      const int rows = min(16, p.group - hblk * 16);
      T* o = reinterpret_cast<T*>(p.out) + (int64_t)b * p.o_stride_b;
      for (int idx = threadIdx.x; idx < rows * D; idx += blockDim.x)
        if (idx % D < p.dv)
          o[(int64_t)(kvh * p.group + hblk * 16 + idx / D) * p.o_stride_h + idx % D] = Elem<T>::from_f(0.f);
    }
    return;   // whole CTA leaves
  }
  const int n_tiles = (hi - lo + TILE_KEYS - 1) / TILE_KEYS;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], p.gather ? 32 * GATHER_WARPS : 1);   // gather: one arrival per lane of the producer warps
      mbar_init(&empty_bar[s], CONSUMER_WARPS);
    }
    *abort_flag = 0;
    fence_mbar_init();
  }
  __syncthreads();

  const int rows_valid = min(16, p.group - hblk * 16);   // q-heads handled by this CTA
  const int head0 = kvh * p.group + hblk * 16;

  // per-warp running state (consumer warps only)
  float m_run[2] = {-CUDART_INF_F, -CUDART_INF_F};
  float l_run[2] = {0.f, 0.f};
  float oacc[NT][4];
#pragma unroll
  for (int t = 0; t < NT; ++t)
#pragma unroll
    for (int j = 0; j < 4; ++j) oacc[t][j] = 0.f;

  if (warp >= CONSUMER_WARPS) {
    // ------------------------------ producer ------------------------------
    // A tile is 64 keys = 64 / min(page, 64) boxes per K/V half; the boxes are spread over the
    // lanes of this warp so that small pages (down to one token per page) still issue quickly.
    if (lane == 0) {
      tma_prefetch_desc(&tmap_k);
      tma_prefetch_desc(&tmap_v);
    }
    if (p.gather) {
      // Pages of fewer than 8 tokens (token-granular caches: page size 1) would need one TMA box of
      // 128 bytes per token and column half, and the copy engine's operation rate, not bandwidth, becomes
      // the limit (measured 0.96 TB/s at page size 1).  Instead the 32 lanes gather 16-byte chunks with
      // cp.async straight into the same 128-byte-swizzled tile layout: 16 lanes per token row, two rows
      // per pass.  The launch has GATHER_WARPS producer warps in this mode, each taking its share of a
      // tile's 64 rows (a producer warp's instruction rate, not bandwidth, is what limits the gather).
      // Everything a lane needs per row is fixed before the tile loop: its 16-byte column of the row (or a
      // zero-length copy past the head size), and the swizzled shared-memory offset of each of its rows.
      // Per row that leaves one shuffle (the row's page), one multiply-add per cache and the two copies.
      constexpr int CHUNKS = D / 8;                 // 16-byte chunks per token row
      constexpr int ROWS_PER_PASS = 32 / CHUNKS;    // 2 (D = 128) or 4 (D = 64)
      constexpr int PASSES = GATHER_ROWS / ROWS_PER_PASS;
      const int c16 = lane % CHUNKS;                // chunk inside the row
      const int sub = lane / CHUNKS;                // row inside the pass
      const int hbox = c16 >> 3, cc = c16 & 7;      // 64-wide column box and chunk inside its 128-byte row
      const int q = warp - CONSUMER_WARPS;
      const bool one_token_pages = p.page_size == 1;
      const bool k_chunk_ok = c16 * 8 < p.dk, v_chunk_ok = c16 * 8 < p.dv;   // chunks past the head size: zeros
      const uint32_t k_bytes = k_chunk_ok ? 16u : 0u, v_bytes = v_chunk_ok ? 16u : 0u;
      const char* k_lane = reinterpret_cast<const char*>(p.k_cache) +
                           ((int64_t)kvh * p.k_stride_head + (k_chunk_ok ? c16 * 8 : 0)) * (int64_t)sizeof(T);
      const char* v_lane = reinterpret_cast<const char*>(p.v_cache) +
                           ((int64_t)kvh * p.v_stride_head + (v_chunk_ok ? c16 * 8 : 0)) * (int64_t)sizeof(T);
      uint32_t row_off[PASSES];
#pragma unroll
      for (int i = 0; i < PASSES; ++i) {
        const int r = q * GATHER_ROWS + sub + i * ROWS_PER_PASS;
        row_off[i] = (uint32_t)(hbox * HALF_BYTES + r * 128 + ((cc ^ (r & 7)) << 4));
      }
      const uint32_t smem_base = smem_u32(smem);
      // (page, slot) of this warp's rows, one row per lane, looked up one tile ahead of the copies
      auto lookup = [&](int t, int& pg, int& sl) {
        const int tok = lo + t * TILE_KEYS + q * GATHER_ROWS + (lane % GATHER_ROWS);
        int page_slot = one_token_pages ? tok : (tok >> p.page_shift);
        if (page_slot >= p.max_pages) page_slot = p.max_pages - 1;   // rows past the table: any valid page
        int page = load_index(p.block_table, (int64_t)b * p.bt_stride + page_slot, p.table_is_int64);
        if (tok >= ctx || page < 0 || page >= p.num_pages) page = 0;  // masked later; keep the address legal
        pg = page;
        sl = tok & (p.page_size - 1);
      };
      int pg, sl;
      lookup(0, pg, sl);
      for (int t = 0; t < n_tiles; ++t) {
        const int s = t % STAGES;
        const uint32_t ph = (t / STAGES) & 1;
        int pg_next = 0, sl_next = 0;
        if (t + 1 < n_tiles) lookup(t + 1, pg_next, sl_next);
        int ok = 1;
        if (lane == 0) ok = mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, 11, t) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (!ok) break;
        const uint32_t stage = smem_base + s * STAGE_BYTES;
#pragma unroll
        for (int i = 0; i < PASSES; ++i) {
          const int rr = sub + i * ROWS_PER_PASS;
          const uint32_t page = (uint32_t)__shfl_sync(0xffffffffu, pg, rr);
          const char* ks = k_lane + (uint64_t)page * p.k_page_bytes;
          const char* vs = v_lane + (uint64_t)page * p.v_page_bytes;
          if (!one_token_pages) {   // uniform
            const uint32_t slot = (uint32_t)__shfl_sync(0xffffffffu, sl, rr);
            ks += (uint64_t)slot * p.k_slot_bytes;
            vs += (uint64_t)slot * p.v_slot_bytes;
          }
          const uint32_t dst = stage + row_off[i];
          cp_async_16_sized<0>(dst, ks, k_bytes);
          cp_async_16_sized<KV_BYTES>(dst, vs, v_bytes);
        }
        cp_async_arrive(&full_bar[s]);
        pg = pg_next;
        sl = sl_next;
      }
    }
    const int keys_per_box = min(p.page_size, TILE_KEYS);
    const int boxes_per_tile = TILE_KEYS / keys_per_box;
    for (int t = 0; !p.gather && warp == CONSUMER_WARPS && t < n_tiles; ++t) {
      const int s = t % STAGES;
      const uint32_t ph = (t / STAGES) & 1;
      int ok = 1;
      if (lane == 0) {
        ok = mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, p.status, 11, t) ? 1 : 0;
        if (ok) mbar_arrive_expect_tx(&full_bar[s], STAGE_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok, 0);
      if (!ok) break;
      uint8_t* kdst = smem + s * STAGE_BYTES;
      uint8_t* vdst = kdst + KV_BYTES;
      const int tok0 = lo + t * TILE_KEYS;
      for (int bx = lane; bx < boxes_per_tile; bx += 32) {
        const int tok = tok0 + bx * keys_per_box;
        int page_slot = tok / p.page_size;
        if (page_slot >= p.max_pages) page_slot = p.max_pages - 1;   // tail boxes past the table: any valid page
        int page = load_index(p.block_table, (int64_t)b * p.bt_stride + page_slot, p.table_is_int64);
        if (tok >= ctx || page < 0 || page >= p.num_pages) page = 0;  // masked later; keep the address legal
        const int slot0 = tok % p.page_size;
#pragma unroll
        for (int h = 0; h < BOXES; ++h) {
          tma_load_4d(kdst + h * HALF_BYTES + bx * keys_per_box * 128, &tmap_k, &full_bar[s], h * 64, kvh, slot0, page);
          tma_load_4d(vdst + h * HALF_BYTES + bx * keys_per_box * 128, &tmap_v, &full_bar[s], h * 64, kvh, slot0, page);
        }
      }
    }
  } else {
    // ------------------------------ consumers ------------------------------
    const int r0 = lane >> 2;        // fragment row (q-head) 0..7, second row is r0 + 8
    const int cq = (lane & 3) * 2;   // fragment column pair
    // Q fragments straight from global memory (rows beyond the group are zero)
    uint32_t qf[KSTEPS][4];
    {
      const T* qb = reinterpret_cast<const T*>(p.q) + (int64_t)b * p.q_stride_b;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int row = r0 + (j & 1) * 8;
          const int col = ks * 16 + cq + (j >> 1) * 8;
          uint32_t v = 0;
          if (row < rows_valid && col < p.dk)
            v = *reinterpret_cast<const uint32_t*>(qb + (int64_t)(head0 + row) * p.q_stride_h + col);
          qf[ks][j] = v;
        }
      }
    }
    const float scale2 = p.sm_scale * 1.4426950408889634f;
    const bool use_cap = p.softcap > 0.f;
    const int mat = lane >> 3;      // ldmatrix: which 8x8 matrix this lane addresses
    const int mrow = lane & 7;

    for (int t = 0; t < n_tiles; ++t) {
      const int s = t % STAGES;
      const uint32_t ph = (t / STAGES) & 1;
      bool ok = mbar_wait(&full_bar[s], ph, abort_flag, p.status, 12, t);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      const uint32_t kbase = smem_u32(smem + s * STAGE_BYTES);
      const uint32_t vbase = kbase + KV_BYTES;
      const int tok0 = lo + t * TILE_KEYS + warp * 16;   // first key of this warp's slice

      // zero V rows past the context so that stale cache bits cannot poison P.V
      if (tok0 + 16 > ctx) {
        for (int i = lane; i < 16 * (D / 8); i += 32) {
          const int key = i / (D / 8);
          if (tok0 + key >= ctx) {
            const int chunk16 = i % (D / 8);
            const int krow = warp * 16 + key;
            uint8_t* dst = smem + s * STAGE_BYTES + KV_BYTES + (chunk16 >> 3) * HALF_BYTES + krow * 128 +
                           (((chunk16 & 7) ^ (krow & 7)) << 4);
            *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
          }
        }
        __syncwarp();
      }

      // ---- S = Q K^T for this warp's 16 keys ----
      float sacc[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int i = 0; i < 4; ++i) sacc[j][i] = 0.f;
#pragma unroll
      for (int ks = 0; ks < KSTEPS; ++ks) {
        const int key = warp * 16 + (mat >> 1) * 8 + mrow;
        const int ch = ks * 2 + (mat & 1);
        const uint32_t addr = kbase + (ch >> 3) * HALF_BYTES + key * 128 + (((ch & 7) ^ (key & 7)) << 4);
        uint32_t b00, b01, b10, b11;
        ldmatrix_x4(addr, b00, b01, b10, b11);
        mma_16816<T>(sacc[0], qf[ks], b00, b01);
        mma_16816<T>(sacc[1], qf[ks], b10, b11);
      }

      // ---- scale, soft-cap, mask, online softmax (base-2 domain) ----
      float mx[2] = {-CUDART_INF_F, -CUDART_INF_F};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int key = tok0 + j * 8 + cq + (i & 1);
          float v = sacc[j][i];
          if (use_cap) v = p.softcap * tanhf(v * p.sm_scale / p.softcap) * 1.4426950408889634f;
          else v *= scale2;
          v = (key < ctx && key >= kv_lo) ? v : -CUDART_INF_F;
          sacc[j][i] = v;
          mx[i >> 1] = fmaxf(mx[i >> 1], v);
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      }
      float alpha[2];
      bool grew = false;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float m_new = fmaxf(m_run[r], mx[r]);
        alpha[r] = (m_new == -CUDART_INF_F) ? 1.f : exp2f(m_run[r] - m_new);
        grew |= (m_new > m_run[r]) && (m_run[r] != -CUDART_INF_F);
        m_run[r] = m_new;
      }
      float psum[2] = {0.f, 0.f};
      uint32_t pf[4];
      {
        float pv[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float mref = m_run[i >> 1];
            const float e = (mref == -CUDART_INF_F) ? 0.f : exp2f(sacc[j][i] - mref);
            pv[j][i] = e;
            psum[i >> 1] += e;
          }
        pf[0] = pack_pair<T>(pv[0][0], pv[0][1]);
        pf[1] = pack_pair<T>(pv[0][2], pv[0][3]);
        pf[2] = pack_pair<T>(pv[1][0], pv[1][1]);
        pf[3] = pack_pair<T>(pv[1][2], pv[1][3]);
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) l_run[r] = l_run[r] * alpha[r] + psum[r];
      if (__any_sync(0xffffffffu, grew)) {
#pragma unroll
        for (int tt = 0; tt < NT; ++tt) {
          oacc[tt][0] *= alpha[0];
          oacc[tt][1] *= alpha[0];
          oacc[tt][2] *= alpha[1];
          oacc[tt][3] *= alpha[1];
        }
      }

      // ---- O += P V ----
#pragma unroll
      for (int n = 0; n < D / 16; ++n) {
        const int key = warp * 16 + (mat & 1) * 8 + mrow;
        const int ch = n * 2 + (mat >> 1);
        const uint32_t addr = vbase + (ch >> 3) * HALF_BYTES + key * 128 + (((ch & 7) ^ (key & 7)) << 4);
        uint32_t v00, v01, v10, v11;
        ldmatrix_x4_trans(addr, v00, v01, v10, v11);
        mma_16816<T>(oacc[2 * n], pf, v00, v01);
        mma_16816<T>(oacc[2 * n + 1], pf, v10, v11);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&empty_bar[s]);
    }
    // quad-reduce the row sums (each lane summed its own 4 keys per row)
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
      l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
  }

  // ------------------------------ cross-warp merge ------------------------------
  __syncthreads();   // every TMA write has been consumed; the ring can be reused
  float* red_o = reinterpret_cast<float*>(smem);                       // [warps][16][D]
  float* red_m = red_o + CONSUMER_WARPS * 16 * D;                      // [warps][16]
  float* red_l = red_m + CONSUMER_WARPS * 16;                          // [warps][16]
  if (warp < CONSUMER_WARPS) {
    const int r0 = lane >> 2;
    const int cq = (lane & 3) * 2;
#pragma unroll
    for (int tt = 0; tt < NT; ++tt) {
      float* o0 = red_o + (warp * 16 + r0) * D + tt * 8 + cq;
      float* o1 = red_o + (warp * 16 + r0 + 8) * D + tt * 8 + cq;
      o0[0] = oacc[tt][0];
      o0[1] = oacc[tt][1];
      o1[0] = oacc[tt][2];
      o1[1] = oacc[tt][3];
    }
    if ((lane & 3) == 0) {
      red_m[warp * 16 + r0] = m_run[0];
      red_m[warp * 16 + r0 + 8] = m_run[1];
      red_l[warp * 16 + r0] = l_run[0];
      red_l[warp * 16 + r0 + 8] = l_run[1];
    }
  }
  __syncthreads();
  T* out = reinterpret_cast<T*>(p.out);
  for (int idx = threadIdx.x; idx < rows_valid * D; idx += blockDim.x) {
    const int row = idx / D;
    const int d = idx - row * D;
    float m = -CUDART_INF_F;
#pragma unroll
    for (int w = 0; w < CONSUMER_WARPS; ++w) m = fmaxf(m, red_m[w * 16 + row]);
    float acc = 0.f, l = 0.f;
#pragma unroll
    for (int w = 0; w < CONSUMER_WARPS; ++w) {
      const float mw = red_m[w * 16 + row];
      const float sc = (mw == -CUDART_INF_F) ? 0.f : exp2f(mw - m);
      acc += red_o[(w * 16 + row) * D + d] * sc;
      l += red_l[w * 16 + row] * sc;
    }
    const int head = head0 + row;
    if (p.max_splits == 1) {
      if (d < p.dv)
        out[(int64_t)b * p.o_stride_b + (int64_t)head * p.o_stride_h + d] = Elem<T>::from_f(l > 0.f ? acc / l : 0.f);
    } else {
      float* dst = p.partial + (((int64_t)b * p.hq + head) * p.max_splits + split) * (D + 2);
      dst[d] = acc;
      if (d == 0) {
        dst[D] = m;
        dst[D + 1] = l;
      }
    }
  }
}

// Merge the per-split partials of one (sequence, q-head): D threads.
template <typename T, int D>
__global__ void __launch_bounds__(D) paged_decode_merge_kernel(const DecodeParams p) {
  const int head = blockIdx.x;
  const int b = blockIdx.y;
  const int d = threadIdx.x;
  const int ctx = load_index(p.kv_seqlens, b, p.lens_is_int64);
  T* out = reinterpret_cast<T*>(p.out) + (int64_t)b * p.o_stride_b + (int64_t)head * p.o_stride_h;
  int lo, hi, kv_lo;
  if (!split_range(ctx, p.window, p.chunk, 0, lo, hi, kv_lo)) {
    if (d < p.dv) out[d] = Elem<T>::from_f(0.f);
    return;
  }
  const int n_splits = min(p.max_splits, (ctx - lo + p.chunk - 1) / p.chunk);
  const float* src = p.partial + ((int64_t)b * p.hq + head) * p.max_splits * (D + 2);
  float m = -CUDART_INF_F;
  for (int s = 0; s < n_splits; ++s) m = fmaxf(m, src[s * (D + 2) + D]);
  float acc = 0.f, l = 0.f;
  for (int s = 0; s < n_splits; ++s) {
    const float ms = src[s * (D + 2) + D];
    const float sc = (ms == -CUDART_INF_F) ? 0.f : exp2f(ms - m);
    acc += src[s * (D + 2) + d] * sc;
    l += src[s * (D + 2) + D + 1] * sc;
  }
  if (d < p.dv) out[d] = Elem<T>::from_f(l > 0.f ? acc / l : 0.f);
}

template <typename T, int D>
static int launch_decode(const CUtensorMap& tk, const CUtensorMap& tv, const DecodeParams& p, cudaStream_t stream) {
  using namespace pd;
  constexpr int STAGE_BYTES = 2 * (D / 64) * TILE_KEYS * 128;
  constexpr int RED_BYTES = CONSUMER_WARPS * 16 * (D + 2) * 4;
  constexpr int RING = STAGES * STAGE_BYTES;
  constexpr int SMEM = (RING > RED_BYTES ? RING : RED_BYTES) + 1024 + 128;
  auto kern = paged_decode_split_kernel<T, D>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) {
    set_last_error("paged_decode: cannot raise dynamic shared memory: %s", cudaGetErrorString(e));
    return (int)e;
  }
  const int hblocks = (p.group + 15) / 16;
  dim3 grid(p.max_splits, p.hkv * hblocks, p.batch);
  kern<<<grid, p.gather ? THREADS + 32 * (GATHER_WARPS - 1) : THREADS, SMEM, stream>>>(tk, tv, p);
  DLB_CUDA_LAUNCH_CHECK();
  if (p.max_splits > 1) {
    paged_decode_merge_kernel<T, D><<<dim3(p.hq, p.batch), D, 0, stream>>>(p);
    DLB_CUDA_LAUNCH_CHECK();
  }
  return DLB_OK;
}

}  // namespace dlb

extern "C" int64_t dlb_paged_decode_workspace_floats(int64_t batch, int64_t hq, int64_t head_dim,
                                                     int64_t max_splits) {
  const int64_t width = head_dim <= 64 ? 64 : 128;   // the tile width the kernel runs at
  return max_splits <= 1 ? 0 : batch * hq * max_splits * (width + 2);
}

extern "C" int dlb_paged_decode(const void* q, const void* k_cache, const void* v_cache, void* out,
                                const void* block_table, const void* kv_seqlens, float* partial, int64_t batch,
                                int64_t hq, int64_t hkv, int64_t head_dim, int64_t head_dim_v, int64_t page_size,
                                int64_t num_pages, int64_t max_pages, int64_t q_stride_b, int64_t q_stride_h,
                                int64_t o_stride_b,
                                int64_t o_stride_h, int64_t k_stride_page, int64_t k_stride_slot,
                                int64_t k_stride_head, int64_t v_stride_page, int64_t v_stride_slot,
                                int64_t v_stride_head, int64_t bt_stride, int table_is_int64, int lens_is_int64,
                                int64_t chunk, int64_t max_splits, int64_t window, float sm_scale, float softcap,
                                int dtype, int32_t* status, void* stream) {
  DLB_NVTX("dlb_paged_decode");
  using namespace dlb;
  DLB_CHECK_ARG(dtype == DLB_DTYPE_BF16 || dtype == DLB_DTYPE_F16, DLB_ERR_UNSUPPORTED,
                "paged_decode: dtype %d (need fp16 or bf16)", dtype);
  DLB_CHECK_ARG(head_dim >= 8 && head_dim <= 128 && head_dim % 8 == 0 && head_dim_v >= 8 && head_dim_v <= 128 &&
                    head_dim_v % 8 == 0,
                DLB_ERR_UNSUPPORTED, "paged_decode: head_dim %lld / %lld not supported (multiples of 8 up to 128)",
                (long long)head_dim, (long long)head_dim_v);
  const int width = (head_dim <= 64 && head_dim_v <= 64) ? 64 : 128;
  DLB_CHECK_ARG(batch >= 0 && hq >= 1 && hkv >= 1 && hq % hkv == 0, DLB_ERR_BAD_ARG, "paged_decode: bad head counts");
  DLB_CHECK_ARG(page_size >= 1 && (page_size & (page_size - 1)) == 0, DLB_ERR_UNSUPPORTED,
                "paged_decode: page size %lld must be a power of two", (long long)page_size);
  DLB_CHECK_ARG(chunk >= 64 && chunk % 64 == 0 && chunk % page_size == 0, DLB_ERR_BAD_ARG,
                "paged_decode: chunk %lld must be a multiple of 64 and of the page size", (long long)chunk);
  DLB_CHECK_ARG(max_splits >= 1 && max_splits <= 65535, DLB_ERR_BAD_ARG, "paged_decode: max_splits out of range");
  DLB_CHECK_ARG(max_splits == 1 || partial != nullptr, DLB_ERR_BAD_ARG, "paged_decode: workspace missing");
  DLB_CHECK_ARG(max_pages >= 1 && num_pages >= 1, DLB_ERR_BAD_ARG, "paged_decode: empty block table or cache");
  DLB_CHECK_ARG(batch <= 65535 && hkv * ((hq / hkv + 15) / 16) <= 65535, DLB_ERR_TOO_LARGE,
                "paged_decode: grid too large");
  if (batch == 0) return DLB_OK;
  DLB_CHECK_ARG(q && k_cache && v_cache && out && block_table && kv_seqlens, DLB_ERR_BAD_ARG,
                "paged_decode: null pointer");
  DLB_CHECK_ARG(q_stride_h % 2 == 0 && q_stride_b % 2 == 0 && ((uintptr_t)q & 3) == 0, DLB_ERR_ALIGNMENT,
                "paged_decode: q must be 4-byte aligned with even strides");
  const int box_slots = (int)(page_size < 64 ? page_size : 64);
  CUtensorMap tk, tv;
  int rc = make_tmap_cache(&tk, k_cache, head_dim, hkv, page_size, num_pages, k_stride_page, k_stride_slot,
                           k_stride_head, box_slots);
  if (rc != DLB_OK) return rc;
  rc = make_tmap_cache(&tv, v_cache, head_dim_v, hkv, page_size, num_pages, v_stride_page, v_stride_slot,
                       v_stride_head, box_slots);
  if (rc != DLB_OK) return rc;

  DecodeParams p;
  p.q = q;
  p.out = out;
  p.partial = partial;
  p.block_table = block_table;
  p.kv_seqlens = kv_seqlens;
  p.q_stride_b = q_stride_b;
  p.q_stride_h = q_stride_h;
  p.o_stride_b = o_stride_b;
  p.o_stride_h = o_stride_h;
  p.bt_stride = bt_stride;
  p.batch = (int)batch;
  p.hq = (int)hq;
  p.hkv = (int)hkv;
  p.group = (int)(hq / hkv);
  p.dk = (int)head_dim;
  p.dv = (int)head_dim_v;
  p.page_size = (int)page_size;
  p.max_pages = (int)max_pages;
  p.num_pages = (int)num_pages;
  p.chunk = (int)chunk;
  p.max_splits = (int)max_splits;
  p.window = (int)window;
  p.table_is_int64 = table_is_int64;
  p.lens_is_int64 = lens_is_int64;
  p.sm_scale = sm_scale;
  p.softcap = softcap;
  p.status = status;
  // pages of fewer than 8 tokens are gathered with cp.async (needs 16-byte aligned rows)
  const bool aligned16 = ((uintptr_t)k_cache & 15) == 0 && ((uintptr_t)v_cache & 15) == 0 && k_stride_page % 8 == 0 &&
                         k_stride_slot % 8 == 0 && k_stride_head % 8 == 0 && v_stride_page % 8 == 0 &&
                         v_stride_slot % 8 == 0 && v_stride_head % 8 == 0;
  // (the lanes address rows as page * page_bytes + slot * slot_bytes with 32-bit byte strides and a shift
  // for the page index, so the page size must be 1, 2 or 4 and the strides below 4 GiB)
  const int64_t esz = 2;
  const bool small_strides = k_stride_page * esz < (1LL << 32) && k_stride_slot * esz < (1LL << 32) &&
                             v_stride_page * esz < (1LL << 32) && v_stride_slot * esz < (1LL << 32);
  p.gather = (page_size < 8 && aligned16 && small_strides) ? 1 : 0;   // page sizes are powers of two: 1, 2, 4
  p.k_cache = k_cache;
  p.v_cache = v_cache;
  p.k_stride_head = k_stride_head;
  p.v_stride_head = v_stride_head;
  p.k_page_bytes = (uint32_t)(k_stride_page * esz);
  p.k_slot_bytes = (uint32_t)(k_stride_slot * esz);
  p.v_page_bytes = (uint32_t)(v_stride_page * esz);
  p.v_slot_bytes = (uint32_t)(v_stride_slot * esz);
  p.page_shift = page_size == 4 ? 2 : (page_size == 2 ? 1 : 0);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == DLB_DTYPE_BF16) {
    return width == 128 ? launch_decode<__nv_bfloat16, 128>(tk, tv, p, s)
                        : launch_decode<__nv_bfloat16, 64>(tk, tv, p, s);
  }
  return width == 128 ? launch_decode<__half, 128>(tk, tv, p, s) : launch_decode<__half, 64>(tk, tv, p, s);
}

// ----------------------------------------------------------------------------
// Allocation-free variant: the split-KV workspace lives in a fixed device array
// ----------------------------------------------------------------------------
// Some callers of a decode step cannot allocate device memory around the call:
// a serving engine whose memory pool was sized once at start-up and handed out
// completely to the KV cache, or a host thread that must not enter the allocator
// because an allocation may synchronise the device (or fail) in the middle of a
// latency-critical token loop.  For them the (acc, m, l) partials of the split
// pass live in a file-scope device array instead of a caller-provided buffer.
//
// Limits and rules
//   * the array holds DLB_DECODE_STATIC_FLOATS fp32 values (32 MiB); every GPU
//     that loads this library carries it until the process exits;
//   * a call needs batch * hq * max_splits * (head_dim + 2) floats (0 when
//     max_splits == 1) and is rejected with DLB_ERR_TOO_LARGE beyond the limit;
//   * the first call on each device resolves the array's device address (one
//     cudaGetSymbolAddress with that device current); make that first call
//     before starting any stream capture on the device;
//   * all calls on a device share the array and it keeps the previous call's
//     contents.  Nothing in it has to start at zero: every (sequence, head,
//     split) slot the merge pass reads was written by the split pass of the same
//     call.  Two calls whose kernels overlap on the GPU (different streams) race
//     on it; serialise them.

namespace dlb {
static __device__ __align__(256) float g_decode_scratch[DLB_DECODE_STATIC_FLOATS];

// Device address of g_decode_scratch on the current device.  In host code the symbol's name
// is only a handle, never an address a kernel may use; the address comes from the runtime.
static int decode_scratch_address(float** out) {
  static float* cache[64] = {nullptr};
  static bool ready[64] = {false};
  static std::mutex mu;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    set_last_error("paged_decode_static: cudaGetDevice: %s", cudaGetErrorString(e));
    return (int)e;
  }
  DLB_CHECK_ARG(dev >= 0 && dev < 64, DLB_ERR_UNSUPPORTED, "paged_decode_static: device ordinal %d", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!ready[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress((void**)&p, g_decode_scratch);
    if (e != cudaSuccess || p == nullptr) {
      set_last_error("paged_decode_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return e != cudaSuccess ? (int)e : DLB_ERR_DRIVER;
    }
    cache[dev] = p;
    ready[dev] = true;
  }
  *out = cache[dev];
  return DLB_OK;
}
}  // namespace dlb

extern "C" int dlb_paged_decode_static(const void* q, const void* k_cache, const void* v_cache, void* out,
                                       const void* block_table, const void* kv_seqlens, int64_t batch, int64_t hq,
                                       int64_t hkv, int64_t head_dim, int64_t page_size, int64_t num_pages,
                                       int64_t max_pages, int64_t q_stride_b, int64_t q_stride_h,
                                       int64_t o_stride_b, int64_t o_stride_h, int64_t k_stride_page,
                                       int64_t k_stride_slot, int64_t k_stride_head, int64_t v_stride_page,
                                       int64_t v_stride_slot, int64_t v_stride_head, int64_t bt_stride,
                                       int table_is_int64, int lens_is_int64, int64_t chunk, int64_t max_splits,
                                       int64_t window, float sm_scale, float softcap, int dtype, int32_t* status,
                                       void* stream) {
  DLB_NVTX("dlb_paged_decode_static");
  using namespace dlb;
  DLB_CHECK_ARG(batch >= 0 && hq >= 1 && head_dim >= 1 && max_splits >= 1, DLB_ERR_BAD_ARG,
                "paged_decode_static: bad sizes");
  const int64_t need = dlb_paged_decode_workspace_floats(batch, hq, head_dim, max_splits);
  DLB_CHECK_ARG(need <= DLB_DECODE_STATIC_FLOATS, DLB_ERR_TOO_LARGE,
                "paged_decode_static: needs %lld workspace floats (batch*hq*max_splits*(head_dim+2)) but the static "
                "scratch holds %lld; lower max_splits (larger chunk) or use dlb_paged_decode with your own buffer",
                (long long)need, (long long)DLB_DECODE_STATIC_FLOATS);
  float* scratch = nullptr;
  const int rc = decode_scratch_address(&scratch);
  if (rc != DLB_OK) return rc;
  return dlb_paged_decode(q, k_cache, v_cache, out, block_table, kv_seqlens, scratch, batch, hq, hkv, head_dim,
                          head_dim, page_size, num_pages, max_pages, q_stride_b, q_stride_h, o_stride_b, o_stride_h,
                          k_stride_page, k_stride_slot, k_stride_head, v_stride_page, v_stride_slot, v_stride_head,
                          bt_stride, table_is_int64, lens_is_int64, chunk, max_splits, window, sm_scale, softcap,
                          dtype, status, stream);
}
